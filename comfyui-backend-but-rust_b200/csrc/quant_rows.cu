// Dynamic per-token absmax int8 activation quantizer with the optional ConvRot rotation fused in.
//
// Entry points gpu_quant_rows / gpu_rotate_rows_f32 of the reference (csrc/kernels.cu:271-298, :316-327):
//   v = prologue(x[m, :])                      elementwise prologues; rounding to the activation dtype as there
//   v = R256(v) per 256-wide group             when rotate != 0 (csrc/common.cuh:99-126: four radix-4 stages of
//                                              the regular Hadamard block, each output 0.5*(((+-a+-b)+-c)+-d))
//   scale = max(min(amax, finite_max) * (1/127), 1e-30)      stored fp32
//   q = clamp(rint(T(T(v) / T(scale))), -128, 127)            T = activation dtype (csrc/kernels.cu:241-255)
//
// The kernel is bound by instruction issue, not by HBM, so it is organised around instruction count:
//   - a 256-wide group belongs to 8 consecutive lanes; a lane loads 32 consecutive elements (16-byte loads)
//   - stages 0 and 1 (index bits 0-3) run in registers on packed f32x2 pairs (element i with element i+16)
//   - the group is transposed through a padded per-warp shared-memory buffer; a lane then holds element pairs
//     (2t, 2t+1) + 16 r, r = 0..15, and runs stages 2 and 3 (index bits 4-7) in registers, again on packed pairs
//   - every butterfly adds in the reference's left-to-right order (a - b is fma(b, -1, a): one rounding, the same),
//     so results are bit-identical whichever thread computes them
//   - bf16 prologues of one variable (SiLU, GELU, GELU-tanh, the sigmoid of GATE) are a 65536-entry table built on
//     the device from the very expressions of the reference and read through L1 (staging it in shared memory left
//     room for too few warps and measured slower)
//   - quantization rounds with cvt.rni and packs with saturation; the codes go back through shared memory so that
//     each lane stores 32 contiguous bytes
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace {

enum { PRO_PLAIN = 0, PRO_RMS = 1, PRO_GATE = 2, PRO_SWIGLU = 3, PRO_LAYERNORM = 4, PRO_SILU = 5, PRO_GELU = 6,
       PRO_ADALN = 7, PRO_SITU = 8, PRO_LN_MOD = 9, PRO_LN_AFFINE = 10, PRO_GELU_TANH = 11, PRO_LN_AFFINE_SILU = 12,
       PRO_SITU_FAST = 13 };  // the reference's src/ffi.rs:15-29

enum { LUT_SILU = 0, LUT_GELU = 1, LUT_GELU_TANH = 2, LUT_SIGMOID = 3, LUT_COUNT = 4 };

// bf16 -> bf16 tables of the one-variable prologues: entry b = bf16(act(float(bf16 with bits b)))
__device__ uint16_t g_act_lut[LUT_COUNT][65536];

__global__ void build_lut_kernel(int which) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= 65536) return;
    const float x = __uint_as_float((uint32_t)b << 16);
    float y;
    switch (which) {
        case LUT_SILU: y = silu_f(x); break;
        case LUT_GELU: y = gelu_f(x); break;
        case LUT_GELU_TANH: y = gelu_tanh_f(x); break;
        default: y = sigmoid_f(x); break;
    }
    g_act_lut[which][b] = __bfloat16_as_ushort(__float2bfloat16_rn(y));
}

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
    int nblocks;        // row blocks; CTAs stride over them
    int lut;            // table index of the prologue (read through L1), or -1
    const float* amax_in;   // when set: row maxima to quantize with (rows whose columns are split across devices)
    float* amax_out;        // when set: write each row's maximum here and stop (first pass of the same)
    // normalising prologues
    const float* norm_w;    // RMS / LAYERNORM weight [K] (nullable), LN_AFFINE weight
    const float* norm_b;    // LN_AFFINE bias [K]
    float eps;
    const void* mod_scale;  // [K] in the activation dtype (nullable except ADALN)
    const void* mod_shift;
};

template <int PRO> __host__ __device__ constexpr bool is_ln() { return PRO == PRO_LAYERNORM || PRO == PRO_LN_MOD || PRO == PRO_LN_AFFINE; }
template <int PRO> __host__ __device__ constexpr bool is_norm() { return PRO == PRO_RMS || PRO == PRO_ADALN || is_ln<PRO>(); }
// floats of shared memory a row needs for the sums of a normalising prologue: one partial per thread of the
// reference's block (ceil(K / 1024) warps), 32 warp sums, the total
__host__ __device__ inline int norm_words(int K) { return (((K >> 8) + 3) >> 2) * 32 + 33; }

constexpr int kGroupWords = 304;   // 256 elements + 4 words of padding per 32, rounded so that groups sit 16 banks apart

__device__ __forceinline__ int tpad(int e) { return e + ((e >> 5) << 2); }

template <typename T> __device__ __forceinline__ float finite_max();
template <> __device__ __forceinline__ float finite_max<float>() { return FLT_MAX; }
template <> __device__ __forceinline__ float finite_max<bf16>() { return 3.38953139e38f; }

// 32 consecutive elements -> floats (and, for bf16, their raw 16-bit patterns when a table prologue wants them)
template <typename T> __device__ __forceinline__ void load32(const T* p, float (&v)[32]);
template <> __device__ __forceinline__ void load32<bf16>(const bf16* p, float (&v)[32]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + c);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[8 * c + 2 * i] = __uint_as_float(w[i] << 16);
            v[8 * c + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}
template <> __device__ __forceinline__ void load32<float>(const float* p, float (&v)[32]) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p) + c);
        v[4 * c] = a.x, v[4 * c + 1] = a.y, v[4 * c + 2] = a.z, v[4 * c + 3] = a.w;
    }
}

__device__ __forceinline__ float lut_f(const uint16_t* lut, float x) {   // x holds a bf16 value
    return __uint_as_float((uint32_t)lut[__float_as_uint(x) >> 16] << 16);
}

// Radix-4 butterfly of the regular Hadamard block on packed pairs; outputs in the reference's association:
//   r0 = .5*(((x0+x1)+x2)-x3)  r1 = .5*(((x0+x1)-x2)+x3)  r2 = .5*(((x0-x1)+x2)+x3)  r3 = .5*(((-x0+x1)+x2)+x3)
__device__ __forceinline__ void h4x2(float2& x0, float2& x1, float2& x2, float2& x3) {
    const float2 m1 = make_float2(-1.f, -1.f), hf = make_float2(0.5f, 0.5f);
    const float2 s = __fadd2_rn(x0, x1);
    const float2 d = __ffma2_rn(x1, m1, x0);                         // x0 - x1
    const float2 r0 = __fmul2_rn(hf, __ffma2_rn(x3, m1, __fadd2_rn(s, x2)));
    const float2 r1 = __fmul2_rn(hf, __fadd2_rn(__ffma2_rn(x2, m1, s), x3));
    const float2 r2 = __fmul2_rn(hf, __fadd2_rn(__fadd2_rn(d, x2), x3));
    const float2 r3 = __fmul2_rn(hf, __fadd2_rn(__ffma2_rn(d, m1, x2), x3));   // (-d + x2) + x3
    x0 = r0, x1 = r1, x2 = r2, x3 = r3;
}
// two radix-4 stages over 16 packed values: index bits (0,1) then (2,3) of the position in P
__device__ __forceinline__ void two_stages(float2 (&P)[16]) {
#pragma unroll
    for (int i = 0; i < 16; i += 4) h4x2(P[i], P[i + 1], P[i + 2], P[i + 3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) h4x2(P[i], P[i + 4], P[i + 8], P[i + 12]);
}

// Codes of two values: q = sat8(rint(T(T(v) / T(scale)))). bf16 fast path: both operands of the division carry 8
// significant bits, so the exact quotient is either representable in fp32 or further than 2^-17 (relative) from every
// bf16 rounding boundary; a reciprocal multiply with one correction step then rounds to the same bf16 as the IEEE
// division. cvt.rni + saturating pack equal clamp(rint(.)) except for NaN (0 instead of -128): `nanacc` turns NaN
// (and stays finite otherwise) so the caller can redo such a lane exactly.
template <typename T>
__device__ __forceinline__ uint32_t quant2(float2 v, float st, float rcp, bool fast, float2& nanacc) {
    if (sizeof(T) == 2 && fast) {
        const __nv_bfloat162 ab = __floats2bfloat162_rn(v.x, v.y);
        const uint32_t au = *reinterpret_cast<const uint32_t*>(&ab);
        const float2 a = make_float2(__uint_as_float(au << 16), __uint_as_float(au & 0xffff0000u));
        const float2 q0 = __fmul2_rn(a, make_float2(rcp, rcp));
        const float2 r = __ffma2_rn(q0, make_float2(-st, -st), a);
        const float2 t = __ffma2_rn(r, make_float2(rcp, rcp), q0);
        const __nv_bfloat162 tb = __floats2bfloat162_rn(t.x, t.y);
        const uint32_t tu = *reinterpret_cast<const uint32_t*>(&tb);
        const float tx = __uint_as_float(tu << 16), ty = __uint_as_float(tu & 0xffff0000u);
        nanacc = __ffma2_rn(make_float2(tx, ty), make_float2(0.f, 0.f), nanacc);
        uint32_t packed;
        asm("{\n\t.reg .s32 a, b;\n\t"
            "cvt.rni.s32.f32 a, %1;\n\t"
            "cvt.rni.s32.f32 b, %2;\n\t"
            "cvt.pack.sat.s8.s32.b32 %0, b, a, 0;\n\t}"
            : "=r"(packed)
            : "f"(tx), "f"(ty));
        return packed;   // byte 0 = code of v.x, byte 1 = code of v.y
    }
    const int qx = clamp_rint_i8(rnd<T>(__fdiv_rn(rnd<T>(v.x), st)), -128.f);
    const int qy = clamp_rint_i8(rnd<T>(__fdiv_rn(rnd<T>(v.y), st)), -128.f);
    return (uint32_t)(qx & 0xff) | ((uint32_t)(qy & 0xff) << 8);
}

// 8 consecutive per-column values as floats
__device__ __forceinline__ void load8v(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void load8v(const bf16* p, float (&v)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[2 * i] = __uint_as_float(w[i] << 16), v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
}

// The reference's soft-capped gated activation (csrc/common.cuh:73-91), operation for operation.
__device__ __forceinline__ float stable_tanh_f(float x) {
    const float t = expm1f(__fmul_rn(-2.f, fabsf(x)));
    return copysignf(__fdiv_rn(-t, __fadd_rn(t, 2.f)), x);
}
__device__ __forceinline__ float situ_f(float hidden, float gate) {
    const float a = __fdiv_rn(__fmul_rn(4.f, stable_tanh_f(__fdiv_rn(gate, 4.f))), __fadd_rn(1.f, expf(-gate)));
    return __fmul_rn(a, __fmul_rn(25.f, stable_tanh_f(__fdiv_rn(hidden, 25.f))));
}
__device__ __forceinline__ float tanh_approx_f(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float situ_fast_f(float hidden, float gate) {
    return __fmul_rn(__fdividef(__fmul_rn(4.f, tanh_approx_f(__fmul_rn(gate, 0.25f))), __fadd_rn(1.f, __expf(-gate))),
                     __fmul_rn(25.f, tanh_approx_f(__fmul_rn(hidden, 0.04f))));
}

template <typename T, int PRO, int MAXT>
__global__ void __launch_bounds__(MAXT) quant_rows_kernel(const QuantArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint16_t* lut = g_act_lut[p.lut >= 0 ? p.lut : 0];
    uint8_t* after_lut = smem;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* tbuf = reinterpret_cast<float*>(after_lut) + (warp * 4 + (lane >> 3)) * kGroupWords;   // this group's buffer
    unsigned* amax_s = reinterpret_cast<unsigned*>(after_lut + (size_t)nwarps * 4 * kGroupWords * 4);   // [3][rows]

    float* norm_s = reinterpret_cast<float*>(amax_s + 3 * p.rows_per_cta);   // [rows][norm_words(K)], normalising prologues only

    for (int i = threadIdx.x; i < 3 * p.rows_per_cta; i += blockDim.x) amax_s[i] = 0u;
    __syncthreads();

    const int tpr = p.tpr;
    const int rloc = threadIdx.x / tpr;               // row inside the CTA
    const int tin = threadIdx.x - rloc * tpr;         // thread inside the row
    const int grp = tin >> 3, t8 = tin & 7;
    int it = 0;
    for (int blk = blockIdx.x; blk < p.nblocks; blk += gridDim.x, ++it) {
        const int64_t m_raw = (int64_t)blk * p.rows_per_cta + rloc;
        const bool live = m_raw < p.M;
        const int64_t m = live ? m_raw : p.M - 1;      // idle rows recompute the last row and store nothing
        const int col = (grp << 8) + (t8 << 5);
        const T* x = reinterpret_cast<const T*>(p.x) + m * p.x_stride + col;

        float v[32];
        load32<T>(x, v);
        if (PRO == PRO_GATE) {
            float gg[32];
            load32<T>(reinterpret_cast<const T*>(p.g) + m * p.g_stride + col, gg);
#pragma unroll
            for (int i = 0; i < 32; ++i)
                v[i] = rnd<T>(v[i] * ((sizeof(T) == 2 && p.lut >= 0) ? lut_f(lut, gg[i]) : rnd<T>(sigmoid_f(gg[i]))));
        } else if (PRO == PRO_SWIGLU) {
            float u[32];
            load32<T>(x + p.up_offset, u);
#pragma unroll
            for (int i = 0; i < 32; ++i)
                v[i] = rnd<T>(((sizeof(T) == 2 && p.lut >= 0) ? lut_f(lut, v[i]) : rnd<T>(silu_f(v[i]))) * u[i]);
        } else if (PRO == PRO_SILU || PRO == PRO_GELU || PRO == PRO_GELU_TANH) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (sizeof(T) == 2 && p.lut >= 0) v[i] = lut_f(lut, v[i]);
                else v[i] = rnd<T>(PRO == PRO_SILU ? silu_f(v[i]) : PRO == PRO_GELU ? gelu_f(v[i]) : gelu_tanh_f(v[i]));
            }
        } else if (PRO == PRO_SITU || PRO == PRO_SITU_FAST) {
            float u[32];   // the gate half of the row; the product is not rounded here (csrc/kernels.cu:107-112)
            load32<T>(x + p.up_offset, u);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = PRO == PRO_SITU ? situ_f(v[i], u[i]) : situ_fast_f(v[i], u[i]);
        }

        if constexpr (is_norm<PRO>()) {
            // Row statistics in the reference's order of additions (csrc/kernels.cu:113-147, csrc/common.cuh:30-55), so
            // that the sums, and everything after them, come out bit for bit: there a block of nwr = ceil(K / 1024)
            // warps holds the row, warp w the groups w, w + nwr, ..., lane l elements 8 l .. 8 l + 7 of each; a thread
            // adds its elements in that order, then a xor-shuffle tree runs over the lanes and another over the warps.
            // Here a thread holds four such 8-runs of one group, so the running sums pass from group to group through
            // shared memory, one round per group of a reference warp.
            const int ngroups = p.K >> 8, nwr = (ngroups + 3) >> 2, words = nwr * 32 + 33;
            const int nrounds = (ngroups + nwr - 1) / nwr;
            float* part = norm_s + rloc * words;
            const int rgi = grp / nwr, rw = grp - rgi * nwr;
            auto row_sum = [&](bool squares) -> float {
                for (int round = 0; round < nrounds; ++round) {
                    if (rgi == round) {
#pragma unroll
                        for (int sub = 0; sub < 4; ++sub) {
                            float* slot = part + rw * 32 + 4 * t8 + sub;
                            float ss = round ? *slot : 0.f;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float e = v[8 * sub + j];
                                ss = squares ? __fmaf_rn(e, e, ss) : __fadd_rn(ss, e);
                            }
                            *slot = ss;
                        }
                    }
                    __syncthreads();
                }
                for (int pi = warp; pi < p.rows_per_cta * nwr; pi += nwarps) {
                    const int row = pi / nwr, ww = pi - row * nwr;
                    float* pr = norm_s + row * words;
                    float t = pr[ww * 32 + lane];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
                    if (lane == 0) pr[nwr * 32 + ww] = t;
                }
                __syncthreads();
                for (int row = warp; row < p.rows_per_cta; row += nwarps) {
                    float* pr = norm_s + row * words;
                    float t = lane < nwr ? pr[nwr * 32 + lane] : 0.f;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
                    if (lane == 0) pr[nwr * 32 + 32] = t;
                }
                __syncthreads();
                return part[nwr * 32 + 32];
            };
            if constexpr (is_ln<PRO>()) {
                const float mean = __fdiv_rn(row_sum(false), (float)p.K);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __fsub_rn(v[i], mean);
            }
            const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(row_sum(true), (float)p.K), p.eps));
            const T* ms_p = reinterpret_cast<const T*>(p.mod_scale);
            const T* sh_p = reinterpret_cast<const T*>(p.mod_shift);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float ms[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, sh[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, nw[8], nb[8];
                if (ms_p) load8v(ms_p + col + 8 * c, ms), load8v(sh_p + col + 8 * c, sh);
                const bool has_w = p.norm_w != nullptr;
                if (has_w) load8v(p.norm_w + col + 8 * c, nw);
                if (PRO == PRO_LN_AFFINE) load8v(p.norm_b + col + 8 * c, nb);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float n = __fmul_rn(v[8 * c + j], rstd);
                    if (PRO == PRO_ADALN) {          // one rounding
                        n = rnd<T>(__fmaf_rn(n, __fadd_rn(1.f, ms[j]), sh[j]));
                    } else if (PRO == PRO_LN_MOD) {  // one rounding after the norm, one after the multiply-add
                        n = rnd<T>(__fmaf_rn(rnd<T>(n), rnd<T>(__fadd_rn(1.f, ms[j])), sh[j]));
                    } else if (PRO == PRO_LN_AFFINE) {
                        n = rnd<T>(__fmaf_rn(n, nw[j], nb[j]));
                    } else {                          // RMS, LAYERNORM: every step rounded
                        if (has_w) n = __fmul_rn(n, nw[j]);
                        n = rnd<T>(n);
                        if (ms_p) {
                            const float a = rnd<T>(__fadd_rn(1.f, ms[j]));
                            // f32 rows: nothing rounds between the product and the sum, and whether they fuse into one
                            // multiply-add is the compiler's choice. In the reference as nvcc 12.9 builds it, LAYERNORM
                            // fuses everywhere and RMS only in the last of its four unrolled group iterations (found by
                            // comparing outputs); that build is what these results are pinned to.
                            if (sizeof(T) == 4 && (PRO == PRO_LAYERNORM || rgi == 3)) n = __fmaf_rn(a, n, sh[j]);
                            else n = rnd<T>(__fadd_rn(rnd<T>(__fmul_rn(a, n)), sh[j]));
                        }
                    }
                    v[8 * c + j] = n;
                }
            }
        }

        float2 P[16];
        if (p.rotate) {
            // stages 0, 1 on the lane's two runs of 16, packed as (element i, element i + 16)
#pragma unroll
            for (int i = 0; i < 16; ++i) P[i] = make_float2(v[i], v[i + 16]);
            two_stages(P);
            // transpose inside the group: lane t8 wrote elements 32 t8 + i, now takes (2 t8, 2 t8 + 1) + 16 r
            const int wbase = tpad(t8 << 5);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                tbuf[wbase + i] = P[i].x;
                tbuf[wbase + 16 + i] = P[i].y;   // element 32 t8 + 16 + i: same 32-run, no pad in between
            }
            __syncwarp();
#pragma unroll
            for (int r = 0; r < 16; ++r) P[r] = *reinterpret_cast<const float2*>(tbuf + tpad(2 * t8 + 16 * r));
            two_stages(P);   // index bits 4-7 = r
            __syncwarp();
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) P[i] = make_float2(v[2 * i], v[2 * i + 1]);   // natural order
        }

        if (p.out_f) {   // gpu_rotate_rows_f32: always rotated, so P holds (2 t8, 2 t8 + 1) + 16 r
            if (live) {
                float* o = p.out_f + m * (int64_t)p.K + (grp << 8) + 2 * t8;
#pragma unroll
                for (int r = 0; r < 16; ++r) *reinterpret_cast<float2*>(o + 16 * r) = P[r];
            }
            continue;
        }

        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fmaxf(fabsf(P[i].x), fabsf(P[i].y)));
        // the group's 8 lanes first, then one shared-memory atomic per group (non-negative floats order as integers)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        unsigned* slot = amax_s + (it % 3) * p.rows_per_cta + rloc;
        if (t8 == 0) atomicMax(slot, __float_as_uint(amax));
        __syncthreads();
        amax = __uint_as_float(*slot);
        amax_s[((it + 2) % 3) * p.rows_per_cta + rloc] = 0u;   // next use is two barriers away, last use one barrier back
        if (p.amax_out) {
            if (live && tin == 0) p.amax_out[m] = amax;
            continue;
        }
        if (p.amax_in) amax = p.amax_in[m];

        const float scale = fmaxf(fminf(amax, finite_max<T>()) * (1.f / 127.f), 1.0e-30f);
        if (live && tin == 0) p.scales[m] = scale;
        const float st = rnd<T>(scale);
        const bool fast = sizeof(T) == 2 && amax <= FLT_MAX;   // rows holding an infinity keep the IEEE division
        const float rcp = fast ? __frcp_rn(st) : 0.f;
        float2 nanacc = make_float2(0.f, 0.f);
        uint32_t c16[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) c16[i] = quant2<T>(P[i], st, rcp, fast, nanacc);
        if (fast && (nanacc.x != nanacc.x || nanacc.y != nanacc.y)) {   // a NaN in this lane: redo it with exact clamping
#pragma unroll
            for (int i = 0; i < 16; ++i) c16[i] = quant2<T>(P[i], st, rcp, false, nanacc);
        }
        int8_t* q = p.q + m * (int64_t)p.K + col;
        if (p.rotate) {
            // codes of (2 t8, 2 t8 + 1) + 16 r back through the group's buffer, so each lane stores 32 contiguous bytes
            uint16_t* cb = reinterpret_cast<uint16_t*>(tbuf);
#pragma unroll
            for (int r = 0; r < 16; ++r) cb[t8 + 8 * r] = (uint16_t)c16[r];
            __syncwarp();
            const uint4 lo = reinterpret_cast<const uint4*>(tbuf)[2 * t8], hi = reinterpret_cast<const uint4*>(tbuf)[2 * t8 + 1];
            __syncwarp();
            if (live) {
                reinterpret_cast<uint4*>(q)[0] = lo;
                reinterpret_cast<uint4*>(q)[1] = hi;
            }
        } else if (live) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = (c16[2 * i] & 0xffffu) | (c16[2 * i + 1] << 16);
            reinterpret_cast<uint4*>(q)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(q)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------------------
struct LutState {
    std::mutex mu;
    bool launched[LUT_COUNT] = {};
    bool done[LUT_COUNT] = {};
    cudaEvent_t ev[LUT_COUNT] = {};
};
LutState g_lut_state[64];

// Makes table `which` of the current device usable by work enqueued on `st` afterwards. The first call per device
// and table launches the builder on `st` (so it should come before any stream capture); later calls on other
// streams are ordered behind it until it is known complete.
int ensure_lut(int which, cudaStream_t st) {
    int dev = 0;
    cudaGetDevice(&dev);
    LutState& s = g_lut_state[dev & 63];
    std::lock_guard<std::mutex> lk(s.mu);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) (void)cudaGetLastError();
    if (cap != cudaStreamCaptureStatusNone) {
        // While a graph is being captured neither event queries nor waits on outside events are allowed. A table
        // requested first inside a capture is built by the captured graph itself, every replay (idempotent); one
        // launched before is taken as complete: the warm-up call that launched it precedes the capture.
        if (!s.launched[which]) {
            build_lut_kernel<<<256, 256, 0, st>>>(which);
            KCHECK();
        }
        return 0;
    }
    if (!s.launched[which]) {
        build_lut_kernel<<<256, 256, 0, st>>>(which);
        KCHECK();
        cudaError_t e = cudaEventCreateWithFlags(&s.ev[which], cudaEventDisableTiming);
        if (e != cudaSuccess) return (int)e;
        e = cudaEventRecord(s.ev[which], st);
        if (e != cudaSuccess) return (int)e;
        s.launched[which] = true;
        return 0;
    }
    if (!s.done[which]) {
        if (cudaEventQuery(s.ev[which]) == cudaSuccess) s.done[which] = true;
        else {
            const cudaError_t e = cudaStreamWaitEvent(st, s.ev[which], 0);
            if (e != cudaSuccess) return (int)e;
        }
    }
    return 0;
}

}  // namespace

// Device address of the bf16 -> bf16 table of a GEMM-epilogue activation (epilogue.cuh's Act codes), built on first use
// like the quantizer's own: the epilogue's out(act(out(v))) on bf16 outputs is a function of 16 bits.
int act_lut_ptr(int act, cudaStream_t st, const uint16_t** out) {
    const int which = act == 1 ? LUT_GELU_TANH : act == 2 ? LUT_SILU : act == 3 ? LUT_GELU : -1;
    if (which < 0) return -204;
    if (int rc = ensure_lut(which, st)) return rc;
    static const uint16_t* base[64];
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(mu);
    const uint16_t*& b = base[dev & 63];
    if (!b) {
        void* addr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&addr, g_act_lut);
        if (e != cudaSuccess) return (int)e;
        b = reinterpret_cast<const uint16_t*>(addr);
    }
    *out = b + (size_t)which * 65536;
    return 0;
}

namespace {

template <typename T, int PRO, int MAXT>
int launch_cfg(QuantArgs& p, int threads, size_t smem, int grid, cudaStream_t st) {
    auto kern = quant_rows_kernel<T, PRO, MAXT>;
    static std::atomic<uint64_t> configured{0};
    if (smem > 48 * 1024) {
        int dev = 0;
        cudaGetDevice(&dev);
        const uint64_t bit = 1ull << (dev & 63);
        if (!(configured.load(std::memory_order_acquire) & bit)) {
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return (int)e;
            configured.fetch_or(bit, std::memory_order_release);
        }
    }
    kern<<<grid, threads, smem, st>>>(p);
    KCHECK();
    return 0;
}

template <typename T, int PRO>
int launch_quant(QuantArgs& p, cudaStream_t st) {
    p.tpr = p.K / 32;
    if (p.tpr > 1024) return -2;  // the reference's limit: K <= 32768 (csrc/kernels.cu:264)
    if (p.M <= 0) return 0;
    static const bool lut_off = [] { const char* e = getenv("GPU_KERNELS_QUANT_LUT"); return e && e[0] == '0'; }();
    int lut = -1;
    if (sizeof(T) == 2 && !lut_off && (int64_t)p.M * p.K >= (1 << 20)) {
        lut = PRO == PRO_SILU || PRO == PRO_SWIGLU ? LUT_SILU : PRO == PRO_GELU ? LUT_GELU : PRO == PRO_GELU_TANH ? LUT_GELU_TANH
              : PRO == PRO_GATE ? LUT_SIGMOID : -1;
    }
    if (lut >= 0) {
        if (int rc = ensure_lut(lut, st)) return rc;
    }
    p.lut = lut;
    const int gcd32 = p.tpr % 32 == 0 ? 32 : (p.tpr % 16 == 0 ? 16 : 8);
    const int r0 = 32 / gcd32;    // rows that make the CTA a whole number of warps
    const int target = 256;
    int rows = r0 * (target / (p.tpr * r0) > 0 ? target / (p.tpr * r0) : 1);
    p.rows_per_cta = rows;
    p.nblocks = (p.M + rows - 1) / rows;
    const int threads = rows * p.tpr;
    const size_t smem = (size_t)(threads / 32) * 4 * kGroupWords * 4 + 3 * rows * 4 +
                        (is_norm<PRO>() ? (size_t)rows * norm_words(p.K) * 4 : 0);
    const int grid = p.nblocks;
    if (threads > 512) return launch_cfg<T, PRO, 1024>(p, threads, smem, grid, st);
    return launch_cfg<T, PRO, 512>(p, threads, smem, grid, st);
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
        case PRO_SITU: return launch_quant<T, PRO_SITU>(p, st);
        case PRO_SITU_FAST: return launch_quant<T, PRO_SITU_FAST>(p, st);
        case PRO_RMS: return launch_quant<T, PRO_RMS>(p, st);
        case PRO_LAYERNORM: return launch_quant<T, PRO_LAYERNORM>(p, st);
        case PRO_LN_MOD: return launch_quant<T, PRO_LN_MOD>(p, st);
        case PRO_ADALN: return p.mod_scale && p.mod_shift ? launch_quant<T, PRO_ADALN>(p, st) : -3;
        // LN_AFFINE needs the bias that only gpu_quant_rows_b carries (the reference reads a null pointer there)
        case PRO_LN_AFFINE: return p.norm_w && p.norm_b ? launch_quant<T, PRO_LN_AFFINE>(p, st) : -3;
        default: return -3;
    }
}

}  // namespace

// Same contract as the reference's gpu_quant_rows (csrc/kernels.cu:271-298): K % 256 == 0 (-1), K <= 32768 (-2),
// known prologue (-3), dtype bf16 or f32 (-4); rows of x start 16-byte aligned.
GPU_API int gpu_quant_rows(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                           int64_t up_offset, const float* norm_w, float eps, const void* mod_scale, const void* mod_shift,
                           int8_t* q, float* scales, int M, int K, int rotate, void* stream) {
    if ((K % 256) != 0) return -1;
    QuantArgs p{x, x_stride, g, g_stride, up_offset, q, scales, nullptr, M, K, rotate, 0, 0, 0, -1, nullptr, nullptr,
                norm_w, nullptr, eps, mod_scale, mod_shift};
    if (dtype == DT_BF16) return dispatch_prologue<bf16>(prologue, p, (cudaStream_t)stream);
    if (dtype == DT_F32) return dispatch_prologue<float>(prologue, p, (cudaStream_t)stream);
    return -4;
}

// gpu_quant_rows with a LayerNorm bias (csrc/kernels.cu:301-314): bf16 only (-4), prologues LN_MOD and LN_AFFINE (-3).
GPU_API int gpu_quant_rows_b(int dtype, int prologue, const void* x, int64_t x_stride, const float* norm_w, const float* norm_b,
                             float eps, const void* mod_scale, const void* mod_shift, int8_t* q, float* scales, int M, int K,
                             int rotate, void* stream) {
    if ((K % 256) != 0) return -1;
    if (dtype != DT_BF16) return -4;
    if (prologue != PRO_LN_MOD && prologue != PRO_LN_AFFINE) return -3;
    QuantArgs p{x, x_stride, nullptr, 0, 0, q, scales, nullptr, M, K, rotate, 0, 0, 0, -1, nullptr, nullptr,
                norm_w, norm_b, eps, mod_scale, mod_shift};
    return dispatch_prologue<bf16>(prologue, p, (cudaStream_t)stream);
}

// Prologue + rotation, fp32 rows out (the weight-only int8 path's activation side; csrc/kernels.cu:316-327).
GPU_API int gpu_rotate_rows_f32(int prologue, const float* x, int64_t x_stride, int64_t up_offset, const float* norm_w,
                                float eps, float* out, int M, int K, void* stream) {
    if ((K % 256) != 0) return -1;
    QuantArgs p{x, x_stride, nullptr, 0, up_offset, nullptr, nullptr, out, M, K, 1, 0, 0, 0, -1, nullptr, nullptr,
                norm_w, nullptr, eps, nullptr, nullptr};
    switch (prologue) {
        case PRO_PLAIN: return launch_quant<float, PRO_PLAIN>(p, (cudaStream_t)stream);
        case PRO_RMS: return launch_quant<float, PRO_RMS>(p, (cudaStream_t)stream);
        case PRO_SWIGLU: return launch_quant<float, PRO_SWIGLU>(p, (cudaStream_t)stream);
        default: return -3;
    }
}

// New, for rows whose K columns are split across devices (row-parallel linears): the per-token scale must come from
// the maximum over the whole row, so quantization runs in two passes around a max-reduction between the devices.
//   pass 1  gpu_quant_rows_amax: prologue + rotation of the local columns, row maxima -> amax [M] (f32)
//   pass 2  gpu_quant_rows_scaled: the same, quantized with the given (reduced) maxima; `scales` receives the scale
// With the reduced maxima the codes equal the corresponding columns of the single-device result bit for bit.
GPU_API int gpu_quant_rows_amax(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                                int64_t up_offset, float* amax, int M, int K, int rotate, void* stream) {
    if ((K % 256) != 0) return -1;
    QuantArgs p{x, x_stride, g, g_stride, up_offset, nullptr, nullptr, nullptr, M, K, rotate, 0, 0, 0, -1, nullptr, amax};
    if (dtype == DT_BF16) return dispatch_prologue<bf16>(prologue, p, (cudaStream_t)stream);
    if (dtype == DT_F32) return dispatch_prologue<float>(prologue, p, (cudaStream_t)stream);
    return -4;
}
GPU_API int gpu_quant_rows_scaled(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                                  int64_t up_offset, const float* amax, int8_t* q, float* scales, int M, int K, int rotate,
                                  void* stream) {
    if ((K % 256) != 0) return -1;
    QuantArgs p{x, x_stride, g, g_stride, up_offset, q, scales, nullptr, M, K, rotate, 0, 0, 0, -1, amax, nullptr};
    if (dtype == DT_BF16) return dispatch_prologue<bf16>(prologue, p, (cudaStream_t)stream);
    if (dtype == DT_F32) return dispatch_prologue<float>(prologue, p, (cudaStream_t)stream);
    return -4;
}
