// Dynamic per-token absmax int8 activation quantizer with the optional ConvRot rotation fused in.
//
// Entry points gpu_quant_rows / gpu_rotate_rows_f32 of the reference (csrc/kernels.cu:271-298, :316-327):
//   v = prologue(x[m, :])                      elementwise prologues; rounding to the activation dtype as there
//   v = R256(v) per 256-wide group             when rotate != 0 (csrc/common.cuh:99-126: four radix-4 stages of
//                                              the regular Hadamard block, each output 0.5*(((+-a+-b)+-c)+-d))
//   scale = max(min(amax, finite_max) * (1/127), 1e-30)      stored fp32
//   q = clamp(rint(T(T(v) / T(scale))), -128, 127)            T = activation dtype (csrc/kernels.cu:241-255)
//
// Layout of the work: a 256-wide group belongs to 8 consecutive lanes; each lane holds four 8-element chunks
// (16-byte loads) in registers. Of the eight index bits of an element inside its group, bits 0-2 are the position
// in the chunk, bits 4 and 6 select the chunk, bits 3, 5 and 7 select the lane. Stage 0 (bits 0,1) runs inside a
// lane; stages 1-3 each pair one register bit with one lane bit, so a lane sends two values to its partner
// (one shuffle per element and stage) and computes the two butterfly outputs that it keeps. Every butterfly adds
// in the reference's order, so the result is bit-identical whichever thread computes it. The row maximum goes
// through shared memory once. No shared-memory staging of the row, no second pass over global memory.
#include "common.cuh"

namespace {

enum { PRO_PLAIN = 0, PRO_RMS = 1, PRO_GATE = 2, PRO_SWIGLU = 3, PRO_LAYERNORM = 4, PRO_SILU = 5, PRO_GELU = 6,
       PRO_ADALN = 7, PRO_SITU = 8, PRO_LN_MOD = 9, PRO_LN_AFFINE = 10, PRO_GELU_TANH = 11, PRO_LN_AFFINE_SILU = 12,
       PRO_SITU_FAST = 13 };  // the reference's src/ffi.rs:15-29

struct QuantArgs {
    const void* x;
    int64_t x_stride;   // elements between rows
    const void* g;      // PRO_GATE: gate logits
    int64_t g_stride;
    int64_t up_offset;  // PRO_SWIGLU: column of `up` inside the x row
    int8_t* q;          // [M, K]
    float* scales;      // [M]
    float* out_f;       // when set: write the rotated fp32 rows here instead of quantizing
    int M, K;
    int rotate;
    int tpr;            // threads per row = K / 32
    int rows_per_cta;
};

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}

template <typename T> __device__ __forceinline__ float finite_max();
template <> __device__ __forceinline__ float finite_max<float>() { return FLT_MAX; }
template <> __device__ __forceinline__ float finite_max<bf16>() { return 3.38953139e38f; }

// One radix-4 stage whose four inputs sit in two registers (a0, a1: register bit 0/1) of two lanes (lane bit
// b = 0/1, partner = lane ^ LX). x0 = (reg 0, lane 0), x1 = (reg 1, lane 0), x2 = (reg 0, lane 1), x3 = (reg 1, lane 1).
// Lane 0 keeps rows 0 and 1 of the block, lane 1 rows 2 and 3:
//   row 0 = ((x0+x1)+x2)-x3   row 1 = ((x0+x1)-x2)+x3   row 2 = ((x0-x1)+x2)+x3   row 3 = ((-x0+x1)+x2)+x3
// With T = X+Y: lane 0 has X=x0, Y=x1, U=x2, V=-x3 and lane 1 has X=x0, Y=-x1, U=x2, V=x3; then
// (T+U)+V is row 0 or row 2, and (T-U)-V is row 1 or minus row 3 (negation commutes with rounding).
template <int LX>
__device__ __forceinline__ void mixed_stage(float& a0, float& a1, bool b, float half_lo, float half_hi) {
    const float p0 = __shfl_xor_sync(0xffffffffu, a0, LX);
    const float p1 = __shfl_xor_sync(0xffffffffu, a1, LX);
    const float X = b ? p0 : a0;
    const float Y = b ? -p1 : a1;
    const float U = b ? a0 : p0;
    const float V = b ? a1 : -p1;
    const float Tt = __fadd_rn(X, Y);
    a0 = __fmul_rn(half_lo, __fadd_rn(__fadd_rn(Tt, U), V));
    a1 = __fmul_rn(half_hi, __fsub_rn(__fsub_rn(Tt, U), V));
}

// R256 of the group held by 8 lanes x v[4][8]. lane8 = lane index inside the group's 8 lanes.
__device__ __forceinline__ void rotate256(float (&v)[4][8], int lane8) {
    // stage 0: index bits 0,1 -- both inside a chunk
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
#pragma unroll
        for (int h = 0; h < 8; h += 4) {
            const float x0 = v[qd][h], x1 = v[qd][h + 1], x2 = v[qd][h + 2], x3 = v[qd][h + 3];
            const float s = __fadd_rn(x0, x1), d = __fsub_rn(x0, x1);
            v[qd][h] = __fmul_rn(0.5f, __fsub_rn(__fadd_rn(s, x2), x3));
            v[qd][h + 1] = __fmul_rn(0.5f, __fadd_rn(__fsub_rn(s, x2), x3));
            v[qd][h + 2] = __fmul_rn(0.5f, __fadd_rn(__fadd_rn(d, x2), x3));
            v[qd][h + 3] = __fmul_rn(0.5f, __fadd_rn(__fadd_rn(-d, x2), x3));
        }
    }
    // stage 1: index bit 2 (position in chunk, bit 2) with bit 3 (lane bit 0)
    {
        const bool b = lane8 & 1;
        const float hl = 0.5f, hh = b ? -0.5f : 0.5f;
#pragma unroll
        for (int qd = 0; qd < 4; ++qd)
#pragma unroll
            for (int j = 0; j < 4; ++j) mixed_stage<1>(v[qd][j], v[qd][j + 4], b, hl, hh);
    }
    // stage 2: index bit 4 (chunk bit 0) with bit 5 (lane bit 1)
    {
        const bool b = (lane8 >> 1) & 1;
        const float hl = 0.5f, hh = b ? -0.5f : 0.5f;
#pragma unroll
        for (int qh = 0; qh < 4; qh += 2)
#pragma unroll
            for (int j = 0; j < 8; ++j) mixed_stage<2>(v[qh][j], v[qh + 1][j], b, hl, hh);
    }
    // stage 3: index bit 6 (chunk bit 1) with bit 7 (lane bit 2)
    {
        const bool b = (lane8 >> 2) & 1;
        const float hl = 0.5f, hh = b ? -0.5f : 0.5f;
#pragma unroll
        for (int ql = 0; ql < 2; ++ql)
#pragma unroll
            for (int j = 0; j < 8; ++j) mixed_stage<4>(v[ql][j], v[ql + 2][j], b, hl, hh);
    }
}

// Element offset, inside its 256-group, of chunk qd of lane lane8 (8 consecutive elements from there).
__device__ __forceinline__ int chunk_offset(int lane8, int qd) {
    return 8 * (lane8 & 1) + 16 * (qd & 1) + 32 * ((lane8 >> 1) & 1) + 64 * (qd >> 1) + 128 * (lane8 >> 2);
}

template <typename T, int PRO>
__global__ void __launch_bounds__(1024) quant_rows_kernel(const QuantArgs p) {
    __shared__ unsigned amax_s[128];
    const int tpr = p.tpr;
    const int rloc = threadIdx.x / tpr;               // row inside the CTA
    const int tin = threadIdx.x - rloc * tpr;         // thread inside the row
    const int64_t m_raw = (int64_t)blockIdx.x * p.rows_per_cta + rloc;
    const bool live = m_raw < p.M;
    const int64_t m = live ? m_raw : p.M - 1;          // idle rows recompute the last row and store nothing
    const int grp = tin >> 3, lane8 = tin & 7;
    const T* x = reinterpret_cast<const T*>(p.x) + m * p.x_stride + (grp << 8);

    if (threadIdx.x < 128) amax_s[threadIdx.x] = 0u;

    float v[4][8];
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
        const int c = chunk_offset(lane8, qd);
        load8<T>(x + c, v[qd]);
        if (PRO == PRO_GATE) {
            float gg[8];
            load8<T>(reinterpret_cast<const T*>(p.g) + m * p.g_stride + (grp << 8) + c, gg);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[qd][j] = rnd<T>(v[qd][j] * rnd<T>(sigmoid_f(gg[j])));
        } else if (PRO == PRO_SWIGLU) {
            float u[8];
            load8<T>(x + p.up_offset + c, u);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[qd][j] = rnd<T>(rnd<T>(silu_f(v[qd][j])) * u[j]);
        } else if (PRO == PRO_SILU) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[qd][j] = rnd<T>(silu_f(v[qd][j]));
        } else if (PRO == PRO_GELU) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[qd][j] = rnd<T>(gelu_f(v[qd][j]));
        } else if (PRO == PRO_GELU_TANH) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[qd][j] = rnd<T>(gelu_tanh_f(v[qd][j]));
        }
    }

    if (p.rotate) rotate256(v, lane8);

    if (p.out_f) {
        if (live) {
            float* o = p.out_f + m * (int64_t)p.K + (grp << 8);
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const int c = chunk_offset(lane8, qd);
                *reinterpret_cast<float4*>(o + c) = make_float4(v[qd][0], v[qd][1], v[qd][2], v[qd][3]);
                *reinterpret_cast<float4*>(o + c + 4) = make_float4(v[qd][4], v[qd][5], v[qd][6], v[qd][7]);
            }
        }
        return;
    }

    float amax = 0.f;
#pragma unroll
    for (int qd = 0; qd < 4; ++qd)
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[qd][j]));
    // the group's 8 lanes first, then one shared-memory atomic per group (non-negative floats order as integers)
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    __syncthreads();
    if (lane8 == 0) atomicMax(&amax_s[rloc], __float_as_uint(amax));
    __syncthreads();
    amax = __uint_as_float(amax_s[rloc]);

    const float scale = fmaxf(fminf(amax, finite_max<T>()) * (1.f / 127.f), 1.0e-30f);
    if (live && tin == 0) p.scales[m] = scale;
    const float st = rnd<T>(scale);
    // bf16: both operands of the division carry 8 significant bits, so the exact quotient is either representable
    // in fp32 or further than 2^-17 (relative) from every bf16 rounding boundary; a reciprocal multiply with one
    // correction step then rounds to the same bf16 as the IEEE division. Rows holding an infinity keep the division.
    const bool fast = sizeof(T) == 2 && amax <= FLT_MAX;
    const float rcp = fast ? __frcp_rn(st) : 0.f;
    if (!live) return;
    int8_t* q = p.q + m * (int64_t)p.K + (grp << 8);
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float a = rnd<T>(v[qd][j]);
            float t;
            if (fast) {
                const float q0 = __fmul_rn(a, rcp);
                t = __fmaf_rn(__fmaf_rn(-q0, st, a), rcp, q0);
            } else {
                t = __fdiv_rn(a, st);
            }
            const int qi = clamp_rint_i8(rnd<T>(t), -128.f);
            w[j >> 2] |= (uint32_t)(qi & 0xff) << (8 * (j & 3));
        }
        *reinterpret_cast<uint2*>(q + chunk_offset(lane8, qd)) = make_uint2(w[0], w[1]);
    }
}

template <typename T, int PRO>
int launch_quant(QuantArgs& p, cudaStream_t st) {
    p.tpr = p.K / 32;
    if (p.tpr > 1024) return -2;  // the reference's limit: K <= 32768 (csrc/kernels.cu:264)
    if (p.M <= 0) return 0;
    const int gcd32 = p.tpr % 32 == 0 ? 32 : (p.tpr % 16 == 0 ? 16 : 8);
    const int r0 = 32 / gcd32;    // rows that make the CTA a whole number of warps
    int rows = r0 * (256 / (p.tpr * r0) > 0 ? 256 / (p.tpr * r0) : 1);
    if (rows > 128) rows = 128;
    p.rows_per_cta = rows;
    const unsigned grid = (unsigned)((p.M + rows - 1) / rows);
    quant_rows_kernel<T, PRO><<<grid, rows * p.tpr, 0, st>>>(p);
    KCHECK();
    return 0;
}

template <typename T>
int dispatch_prologue(int prologue, QuantArgs& p, cudaStream_t st) {
    switch (prologue) {
        case PRO_PLAIN: return launch_quant<T, PRO_PLAIN>(p, st);
        case PRO_GATE: return launch_quant<T, PRO_GATE>(p, st);
        case PRO_SWIGLU: return launch_quant<T, PRO_SWIGLU>(p, st);
        case PRO_SILU: return launch_quant<T, PRO_SILU>(p, st);
        case PRO_GELU: return launch_quant<T, PRO_GELU>(p, st);
        case PRO_GELU_TANH: return launch_quant<T, PRO_GELU_TANH>(p, st);
        // the normalising prologues (RMS, LAYERNORM, ADALN, SITU, LN_MOD, LN_AFFINE...) are not built yet
        default: return -3;
    }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

// Same contract as the reference's gpu_quant_rows (csrc/kernels.cu:271-298): K % 256 == 0 (-1), K <= 32768 (-2),
// known prologue (-3), dtype bf16 or f32 (-4); rows of x start 16-byte aligned.
GPU_API int gpu_quant_rows(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                           int64_t up_offset, const float* norm_w, float eps, const void* mod_scale, const void* mod_shift,
                           int8_t* q, float* scales, int M, int K, int rotate, void* stream) {
    (void)norm_w, (void)eps, (void)mod_scale, (void)mod_shift;
    if ((K % 256) != 0) return -1;
    QuantArgs p{x, x_stride, g, g_stride, up_offset, q, scales, nullptr, M, K, rotate, 0, 0};
    if (dtype == DT_BF16) return dispatch_prologue<bf16>(prologue, p, (cudaStream_t)stream);
    if (dtype == DT_F32) return dispatch_prologue<float>(prologue, p, (cudaStream_t)stream);
    return -4;
}

// Prologue + rotation, fp32 rows out (the weight-only int8 path's activation side; csrc/kernels.cu:316-327).
GPU_API int gpu_rotate_rows_f32(int prologue, const float* x, int64_t x_stride, int64_t up_offset, const float* norm_w,
                                float eps, float* out, int M, int K, void* stream) {
    (void)norm_w, (void)eps;
    if ((K % 256) != 0) return -1;
    QuantArgs p{x, x_stride, nullptr, 0, up_offset, nullptr, nullptr, out, M, K, 1, 0, 0};
    switch (prologue) {
        case PRO_PLAIN: return launch_quant<float, PRO_PLAIN>(p, (cudaStream_t)stream);
        case PRO_SWIGLU: return launch_quant<float, PRO_SWIGLU>(p, (cudaStream_t)stream);
        default: return -3;
    }
}
