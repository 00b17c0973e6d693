// Dynamic per-token absmax int8 activation quantizer with the optional ConvRot rotation fused in.
//
// Entry points gpu_quant_rows / gpu_rotate_rows_f32 of the reference (csrc/kernels.cu:271-298, :316-327):
//   v = prologue(x[m, :])                      elementwise prologues; rounding to the activation dtype as there
//   v = R256(v) per 256-wide group             when rotate != 0 (csrc/common.cuh:99-126: four radix-4 stages of
//                                              the regular Hadamard block, each output 0.5*(((+-a+-b)+-c)+-d))
//   scale = max(min(amax, finite_max) * (1/127), 1e-30)      stored fp32
//   q = clamp(rint(T(T(v) / T(scale))), -128, 127)            T = activation dtype (csrc/kernels.cu:241-255)
//
// The kernel is bound by instruction issue before HBM, so it is organised around instruction count and around keeping
// the issue slots busy:
//   - without the rotation the kernel is short enough to wait for HBM: persistent CTAs walk row blocks and, while one
//     block is computed, one bulk asynchronous copy per row (cp.async.bulk, completion on an mbarrier) brings the next
//     block's rows into shared memory; with the rotation (arithmetic-bound) each CTA takes one block with direct loads
//   - a 256-wide group belongs to 8 consecutive lanes; a lane takes 32 consecutive elements (16-byte loads)
//   - stages 0 and 1 (index bits 0-3) run in registers on packed f32x2 pairs (element i with element i+16)
//   - the group is transposed through a padded per-warp shared-memory buffer; a lane then holds element pairs
//     (2t, 2t+1) + 16 r, r = 0..15, and runs stages 2 and 3 (index bits 4-7) in registers, again on packed pairs
//   - every butterfly adds in the reference's left-to-right order (a - b is fma(b, -1, a): one rounding, the same),
//     so results are bit-identical whichever thread computes them
//   - bf16 prologues of one variable (SiLU, GELU, GELU-tanh, the sigmoid of GATE) are a 65536-entry table built on
//     the device from the very expressions of the reference and read through L1 (keeping the hot part, 2^-14 <= |x| < 128,
//     in shared memory measured slower: 129 against 101 us at M = 4352, K = 12288, the index arithmetic and the bank
//     conflicts of 32 scattered 2-byte reads cost more than the L1 gather)
//   - the division by the scale is a multiplication by its reciprocal (exact for this purpose, see quant2), the
//     codes are rounded by cvt.rni straight from bf16 and packed with saturation, and go back through shared memory
//     so that each lane stores 32 contiguous bytes
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "epilogue.cuh"

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
    int64_t up_offset;  // PRO_SWIGLU, PRO_SITU*: column of the second half inside the x row
    int8_t* q;          // [M, K]
    float* scales;      // [M]
    float* out_f;       // when set: write the rotated fp32 rows here instead of quantizing
    int M, K;
    int rotate;
    int tpr;            // threads per row = K / 32
    int rows_per_cta;
    int nblocks;        // row blocks; CTAs stride over them
    int lut;            // table index of the prologue, or -1
    const float* amax_in;   // when set: row maxima to quantize with (rows whose columns are split across devices)
    float* amax_out;        // when set: write each row's maximum here and stop (first pass of the same)
    // normalising prologues
    const float* norm_w;    // RMS / LAYERNORM weight [K] (nullable), LN_AFFINE weight
    const float* norm_b;    // LN_AFFINE bias [K]
    float eps;
    const void* mod_scale;  // [K] in the activation dtype (nullable except ADALN)
    const void* mod_shift;
    // shared-memory plan (byte offsets from the dynamic shared memory base), filled in by launch_quant
    int staged;             // rows arrive through the staging buffer (bulk copies) instead of direct loads
    uint32_t off_amax, off_norm, off_stage, off_bar;
    // when set (with out_f unset): the rotated fp32 rows leave as two bf16 rows, hi = bf16(v) and lo = bf16(v - hi)
    bf16* out_hi;
    bf16* out_lo;
};

template <int PRO> __host__ __device__ constexpr bool is_ln() { return PRO == PRO_LAYERNORM || PRO == PRO_LN_MOD || PRO == PRO_LN_AFFINE; }
template <int PRO> __host__ __device__ constexpr bool is_norm() { return PRO == PRO_RMS || PRO == PRO_ADALN || is_ln<PRO>(); }
// prologues that read a second stream per row: the gate logits (GATE) or the other half of the row (SWIGLU, SITU)
template <int PRO> __host__ __device__ constexpr bool has_aux() {
    return PRO == PRO_GATE || PRO == PRO_SWIGLU || PRO == PRO_SITU || PRO == PRO_SITU_FAST;
}
// floats of shared memory a row needs for the sums of a normalising prologue: one partial per thread of the
// reference's block (ceil(K / 1024) warps), 32 warp sums, the total
__host__ __device__ inline int norm_words(int K) { return (((K >> 8) + 3) >> 2) * 32 + 33; }

// Transposition buffers: per 8-lane team 256 elements + 4 words of padding per 32 (288 words), laid out so that every
// shared-memory access of the transposition is free of bank conflicts across the four teams of a warp:
//   - a lane writes element 32 t8 + i as one 32-bit store per i; over a team's lanes these hit banks 4 t8 + i, i.e. one
//     residue class modulo 4. The four teams must cover the four classes: teams 1 and 3 store each element pair swapped
//     (column i ^ 1), teams 2 and 3 start two words later
//   - a lane reads element pairs (2 t8, 2 t8 + 1) + 16 r as 64-bit loads, 16 consecutive banks per team; a half-warp holds
//     two teams, which start 16 banks apart
// Teams 1 and 3 therefore hold their pairs as (odd element, even element) from the transposition on; the codes are
// swapped back when they are written out.
constexpr int kGroupWords = 304;          // team pitch inside a warp: 16 banks (mod 32) apart
constexpr int kWarpWords = 4 * 304 + 32;  // warp pitch: a multiple of 32 words with room for the two-word shift

__device__ __forceinline__ int tpad(int e) { return e + ((e >> 5) << 2); }

template <typename T> __device__ __forceinline__ float finite_max();
template <> __device__ __forceinline__ float finite_max<float>() { return FLT_MAX; }
template <> __device__ __forceinline__ float finite_max<bf16>() { return 3.38953139e38f; }

__device__ __forceinline__ void unpack_bf16x8(const uint4 u, float* v) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
// 32 consecutive elements -> floats, from global memory (read-only path) or from the staging buffer
template <typename T, bool SMEM> __device__ __forceinline__ void load32(const T* p, float (&v)[32]) {
    if constexpr (sizeof(T) == 2) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 u = SMEM ? reinterpret_cast<const uint4*>(p)[c] : __ldg(reinterpret_cast<const uint4*>(p) + c);
            unpack_bf16x8(u, v + 8 * c);
        }
    } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 a = SMEM ? reinterpret_cast<const float4*>(p)[c] : __ldg(reinterpret_cast<const float4*>(p) + c);
            v[4 * c] = a.x, v[4 * c + 1] = a.y, v[4 * c + 2] = a.z, v[4 * c + 3] = a.w;
        }
    }
}

__device__ __forceinline__ float lut_f(const uint16_t* lut, float x) {   // x holds a bf16 value; whole table, global
    return __uint_as_float((uint32_t)__ldg(lut + (__float_as_uint(x) >> 16)) << 16);
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

// max(|a|, |b|, |c|) that is NaN as soon as one input is
__device__ __forceinline__ float max3_abs_nan(float a, float b, float c) {
    float m;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(fabsf(a)), "f"(fabsf(b)), "f"(fabsf(c)));
    return m;
}

// Codes of two values: q = sat8(rint(T(T(v) / T(scale)))).
// bf16 fast path. Both operands of the division carry 8 significant bits: a = A 2^i, st = S 2^j with integers
// A, S < 256. A bf16 rounding boundary is M 2^k with M odd and 256 < M < 512; a quotient equal to one would need
// A 2^n = S M, impossible because the odd part of the left side is below 256 and that of the right side is at least 257.
// So the exact quotient differs from every boundary by at least 1 / (S M) > 2^-17 relative, while a (correctly rounded)
// reciprocal times a is within 2^-23 of it: both round to the same bf16, and no correction step is needed
// (tests/test_quant_division.py enumerates every pair of significands).
// The magic-number rint + saturating pack equal clamp(rint(.)) for finite values; the caller keeps rows that hold a NaN
// or an infinity off this path.
// (the fast path on two values already rounded to bf16, packed in one word)
__device__ __forceinline__ uint32_t quant2_bf16_bits(uint32_t au, float rcp) {
    const float2 a = make_float2(__uint_as_float(au << 16), __uint_as_float(au & 0xffff0000u));
    const float2 t = __fmul2_rn(a, make_float2(rcp, rcp));
    const __nv_bfloat162 tb = __floats2bfloat162_rn(t.x, t.y);
    const uint32_t tu = *reinterpret_cast<const uint32_t*>(&tb);
    // rint by adding 1.5 * 2^23 (round to nearest even at unit spacing, |t| <= 128): the integer sits in the low bits.
    // The float -> integer conversion instructions share a narrow pipe with the bf16 conversions above, and that
    // pipe, not HBM, bounded this kernel; the addition runs on the FP32 pipe instead.
    const float2 u = __fadd2_rn(make_float2(__uint_as_float(tu << 16), __uint_as_float(tu & 0xffff0000u)),
                                make_float2(12582912.f, 12582912.f));
    const int n0 = (int)__float_as_uint(u.x) - 0x4B400000, n1 = (int)__float_as_uint(u.y) - 0x4B400000;
    uint32_t packed;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(packed) : "r"(n1), "r"(n0));
    return packed;   // byte 0 = code of the low half, byte 1 = code of the high half
}
template <typename T>
__device__ __forceinline__ uint32_t quant2(float2 v, float st, float rcp, bool fast) {
    if (sizeof(T) == 2 && fast) {
        const __nv_bfloat162 ab = __floats2bfloat162_rn(v.x, v.y);
        return quant2_bf16_bits(*reinterpret_cast<const uint32_t*>(&ab), rcp);
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
    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(p)), v);
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

// One bulk asynchronous copy, global -> this CTA's shared memory, completion credited to an mbarrier. Both addresses
// 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ int g_quant_status = 0;   // a staging wait that ran out records ST_TIMEOUT_FULL here

// MAXT = 384 asks for two CTAs per SM (at most 80 registers: 768 threads with the next block's rows in flight);
// longer rows take one larger CTA.
template <typename T, int PRO, int MAXT>
__global__ void __launch_bounds__(MAXT, MAXT <= 384 ? 2 : 1) quant_rows_kernel(const QuantArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint16_t* lut = g_act_lut[p.lut >= 0 ? p.lut : 0];
    const unsigned wmask = __activemask();            // the last warp of a CTA may be partial (threads = rows * K / 32)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;   // nwarps: whole warps
    const int team = lane >> 3, tsw = team & 1;        // team of the warp; teams 1 and 3 keep their pairs swapped
    float* tbuf = reinterpret_cast<float*>(smem) + warp * kWarpWords + team * kGroupWords + 4 * (team >> 1);   // this team's buffer
    float* tbuf_w = tbuf - 2 * (team >> 1);            // where its transposition writes and reads start (two words later for teams 2, 3)
    unsigned* amax_s = reinterpret_cast<unsigned*>(smem + p.off_amax);   // [3][rows]
    float* norm_s = reinterpret_cast<float*>(smem + p.off_norm);         // [rows][norm_words(K)], normalising prologues only
    const bool use_lut = sizeof(T) == 2 && p.lut >= 0;
    const uint32_t bar = smem_u32(smem + p.off_bar);
    uint8_t* stage = smem + p.off_stage;              // [x rows | aux rows], one block of rows
    const uint32_t row_bytes = (uint32_t)p.K * sizeof(T);

    for (int i = threadIdx.x; i < 3 * p.rows_per_cta; i += blockDim.x) amax_s[i] = 0u;
    if (p.staged && threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();

    // Staging: the rows of block `blk` (and their second stream) -> the staging buffer, one bulk copy each, issued by
    // the first warp; the barrier's phase completes when all their bytes have landed.
    auto issue_block = [&](int blk) {
        if (warp != 0) return;
        const int64_t m0 = (int64_t)blk * p.rows_per_cta;
        const int live = (int)min((int64_t)p.rows_per_cta, (int64_t)p.M - m0);
        if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)live * row_bytes * (has_aux<PRO>() ? 2u : 1u));
        __syncwarp();
        for (int r = lane; r < live; r += 32) {
            const T* src = reinterpret_cast<const T*>(p.x) + (m0 + r) * p.x_stride;
            bulk_load(smem_u32(stage + (size_t)r * row_bytes), src, row_bytes, bar);
            if (has_aux<PRO>()) {
                const T* aux = PRO == PRO_GATE ? reinterpret_cast<const T*>(p.g) + (m0 + r) * p.g_stride : src + p.up_offset;
                bulk_load(smem_u32(stage + (size_t)(p.rows_per_cta + r) * row_bytes), aux, row_bytes, bar);
            }
        }
    };
    if (p.staged && (int)blockIdx.x < p.nblocks) issue_block(blockIdx.x);

    const int tpr = p.tpr;
    const int rloc = threadIdx.x / tpr;               // row inside the CTA
    const int tin = threadIdx.x - rloc * tpr;         // thread inside the row
    const int grp = tin >> 3, t8 = tin & 7;
    const int col = (grp << 8) + (t8 << 5);
    int it = 0;
    for (int blk = blockIdx.x; blk < p.nblocks; blk += gridDim.x, ++it) {
        const int64_t m_raw = (int64_t)blk * p.rows_per_cta + rloc;
        const bool live = m_raw < p.M;
        const int64_t m = live ? m_raw : p.M - 1;      // idle rows compute on the last row (or on stale staging) and store nothing

        float v[32], u[32];
        if (p.staged) {
            // bounded wait for this block's bytes; on expiry the CTA records the fact and leaves
            bool ok = mbar_try_wait(bar, it & 1);
            if (!ok) {
                const uint64_t t0 = globaltimer_ns();
                for (uint32_t n = 1; !(ok = mbar_try_wait(bar, it & 1)); ++n)
                    if ((n & 255u) == 0u && globaltimer_ns() - t0 > kWaitLimitNs) break;
            }
            if (!ok) {
                atomicCAS(&g_quant_status, 0, ST_TIMEOUT_FULL);
                return;
            }
            const T* xs = reinterpret_cast<const T*>(stage + (size_t)rloc * row_bytes) + col;
            load32<T, true>(xs, v);
            if (has_aux<PRO>()) load32<T, true>(reinterpret_cast<const T*>(stage + (size_t)(p.rows_per_cta + rloc) * row_bytes) + col, u);
            // every thread holds its elements, so the buffer can take the next block; the copy engine writes through the
            // asynchronous proxy, hence the proxy fence between these reads and the barrier that releases the buffer
            fence_proxy_async_smem();
            __syncthreads();
            if (blk + (int)gridDim.x < p.nblocks) issue_block(blk + gridDim.x);
        } else {
            const T* x = reinterpret_cast<const T*>(p.x) + m * p.x_stride + col;
            load32<T, false>(x, v);
            if (PRO == PRO_GATE) load32<T, false>(reinterpret_cast<const T*>(p.g) + m * p.g_stride + col, u);
            else if (has_aux<PRO>()) load32<T, false>(x + p.up_offset, u);
        }

        if (PRO == PRO_GATE || PRO == PRO_SWIGLU || PRO == PRO_SILU || PRO == PRO_GELU || PRO == PRO_GELU_TANH) {
            // v = T(act(a)) [* b]: a is the gate logit (GATE), the row itself otherwise
            float* a = PRO == PRO_GATE ? u : v;
            if (use_lut) {
#pragma unroll
                for (int i = 0; i < 32; ++i) a[i] = lut_f(lut, a[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    a[i] = rnd<T>(PRO == PRO_GATE ? sigmoid_f(a[i]) : (PRO == PRO_SILU || PRO == PRO_SWIGLU) ? silu_f(a[i])
                                  : PRO == PRO_GELU ? gelu_f(a[i]) : gelu_tanh_f(a[i]));
            }
            if (PRO == PRO_GATE || PRO == PRO_SWIGLU) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = rnd<T>(__fmul_rn(v[i], u[i]));
            }
        } else if (PRO == PRO_SITU || PRO == PRO_SITU_FAST) {
            // u = the gate half of the row; the product is not rounded here (csrc/kernels.cu:107-112)
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
                // the two shuffle trees run in whole warps only
                for (int pi = warp; pi < p.rows_per_cta * nwr && warp < nwarps; pi += nwarps) {
                    const int row = pi / nwr, ww = pi - row * nwr;
                    float* pr = norm_s + row * words;
                    float t = pr[ww * 32 + lane];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
                    if (lane == 0) pr[nwr * 32 + ww] = t;
                }
                __syncthreads();
                for (int row = warp; row < p.rows_per_cta && warp < nwarps; row += nwarps) {
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
            float* we = tbuf_w + tpad(t8 << 5) + tsw;     // even columns go one word up in a swapping team,
            float* wo = tbuf_w + tpad(t8 << 5) - tsw;     // odd columns one word down: column i ^ 1
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float* w = (i & 1) ? wo : we;
                w[i] = P[i].x;
                w[16 + i] = P[i].y;   // element 32 t8 + 16 + i: same 32-run, no pad in between
            }
            __syncwarp(wmask);
#pragma unroll
            for (int r = 0; r < 16; ++r) P[r] = *reinterpret_cast<const float2*>(tbuf_w + tpad(2 * t8 + 16 * r));
            two_stages(P);   // index bits 4-7 = r; in a swapping team .x is the odd element of the pair
            __syncwarp(wmask);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) P[i] = make_float2(v[2 * i], v[2 * i + 1]);   // natural order
        }

        if (p.out_hi) {  // the weight-only linear's activation side: rotated rows split into two bf16 terms
            if (live) {
                const int64_t o = m * (int64_t)p.K + (grp << 8) + 2 * t8;
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const float2 v2 = tsw ? make_float2(P[r].y, P[r].x) : P[r];
                    const __nv_bfloat162 h = __floats2bfloat162_rn(v2.x, v2.y);
                    const float2 hf = __bfloat1622float2(h);
                    *reinterpret_cast<__nv_bfloat162*>(p.out_hi + o + 16 * r) = h;
                    *reinterpret_cast<__nv_bfloat162*>(p.out_lo + o + 16 * r) = __floats2bfloat162_rn(__fsub_rn(v2.x, hf.x), __fsub_rn(v2.y, hf.y));
                }
            }
            continue;
        }
        if (p.out_f) {   // gpu_rotate_rows_f32: always rotated, so P holds (2 t8, 2 t8 + 1) + 16 r
            if (live) {
                float* o = p.out_f + m * (int64_t)p.K + (grp << 8) + 2 * t8;
#pragma unroll
                for (int r = 0; r < 16; ++r) *reinterpret_cast<float2*>(o + 16 * r) = tsw ? make_float2(P[r].y, P[r].x) : P[r];
            }
            continue;
        }

        // This thread's maximum. The three-input form propagates a NaN, which the reference's fmaxf drops: a thread that
        // meets one recomputes its maximum without it and takes the exact division below.
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = max3_abs_nan(amax, P[i].x, P[i].y);
        const bool has_nan = amax != amax;
        if (has_nan) {
            amax = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fmaxf(fabsf(P[i].x), fabsf(P[i].y)));
        }
        // the group's 8 lanes first, then one shared-memory atomic per group (non-negative floats order as integers)
        amax = fmaxf(amax, __shfl_xor_sync(wmask, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(wmask, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(wmask, amax, 4));
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
        // rows holding an infinity, and threads holding a NaN, keep the IEEE division and the exact clamp
        const bool fast = sizeof(T) == 2 && amax <= FLT_MAX && !has_nan;
        const float rcp = fast ? __frcp_rn(st) : 0.f;
        uint32_t c16[16];
        if (fast) {      // one branch for the row, not one per pair
#pragma unroll
            for (int i = 0; i < 16; ++i) c16[i] = quant2<T>(P[i], st, rcp, true);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) c16[i] = quant2<T>(P[i], st, rcp, false);
        }
        int8_t* q = p.q + m * (int64_t)p.K + col;
        if (p.rotate) {
            // codes of (2 t8, 2 t8 + 1) + 16 r back through the group's buffer, so each lane stores 32 contiguous bytes
            uint16_t* cb = reinterpret_cast<uint16_t*>(tbuf);
            const uint32_t order = tsw ? 0x3201u : 0x3210u;   // a swapping team puts its two codes back in element order
#pragma unroll
            for (int r = 0; r < 16; ++r) cb[t8 + 8 * r] = (uint16_t)__byte_perm(c16[r], 0u, order);
            __syncwarp(wmask);
            const uint4 lo = reinterpret_cast<const uint4*>(tbuf)[2 * t8], hi = reinterpret_cast<const uint4*>(tbuf)[2 * t8 + 1];
            __syncwarp(wmask);
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

// ---- fp16 (SD / SDXL) flavour ------------------------------------------------------------------------------------------
// The reference's fp16 row quantizer (csrc/sd.cu:578-597) differs from the one above in its rounding points: values are
// rounded to half after the rotation, the row maximum is taken over the rounded values, scale = max(mx, 1e-30) / 127 is
// a division, the divisor is half(scale) unless that underflows, and q = clamp(rint(half(half(v) / st))). Rotation groups
// are 256 (four stages) or 64 (three). Same thread layout as above (32 consecutive elements per lane): 256-groups go
// through the same conflict-free transposition; a 64-group is two neighbouring lanes, whose third stage is one exchange
// of registers. The division is a reciprocal multiply with one Newton step: the exact quotient of two 11-bit significands
// is never on a half rounding boundary and at least 2^-23 (relative) away from one, and the refined product is within
// 2^-24 of it, so both round to the same half (tests/test_quant_division.py enumerates the significand pairs).
template <int ROT>
__global__ void __launch_bounds__(512) sd_quant_fast_kernel(const half* __restrict__ x, int64_t x_stride, int8_t* __restrict__ q,
                                                            float* __restrict__ scales, int M, int K, int tpr, int rows,
                                                            uint32_t off_amax) {
    extern __shared__ __align__(128) uint8_t smem[];
    const unsigned wmask = __activemask();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int team = lane >> 3, tsw = team & 1, t8 = lane & 7;
    float* tbuf = reinterpret_cast<float*>(smem) + warp * kWarpWords + team * kGroupWords + 4 * (team >> 1);
    float* tbuf_w = tbuf - 2 * (team >> 1);
    unsigned* amax_s = reinterpret_cast<unsigned*>(smem + off_amax);
    for (int i = threadIdx.x; i < rows; i += blockDim.x) amax_s[i] = 0u;
    __syncthreads();
    const int rloc = threadIdx.x / tpr, tin = threadIdx.x - rloc * tpr;
    const int64_t m_raw = (int64_t)blockIdx.x * rows + rloc;
    const bool live = m_raw < M;
    const int64_t m = live ? m_raw : M - 1;            // idle rows recompute the last row and store nothing
    const half* r = x + m * x_stride + tin * 32;
    float v[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(r) + c);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[8 * c + 2 * i] = f.x, v[8 * c + 2 * i + 1] = f.y;
        }
    }
    float2 P[16];
    if (ROT) {
#pragma unroll
        for (int i = 0; i < 16; ++i) P[i] = make_float2(v[i], v[i + 16]);
        two_stages(P);                                  // index bits 0-3
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) P[i] = make_float2(v[2 * i], v[2 * i + 1]);
    }
    if (ROT == 256) {
        float* we = tbuf_w + tpad(t8 << 5) + tsw;
        float* wo = tbuf_w + tpad(t8 << 5) - tsw;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float* w = (i & 1) ? wo : we;
            w[i] = P[i].x;
            w[16 + i] = P[i].y;
        }
        __syncwarp(wmask);
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) P[rr] = *reinterpret_cast<const float2*>(tbuf_w + tpad(2 * t8 + 16 * rr));
        two_stages(P);                                  // index bits 4-7
        __syncwarp(wmask);
    } else if (ROT == 64) {
        // third stage, index bits 4 and 5: bit 4 is the pair's half, bit 5 the lane's parity. The even lane holds x0, x1
        // and computes outputs 0 and 1 of the block, the odd lane holds x2, x3 and computes outputs 2 and 3.
        const bool even = (lane & 1) == 0;
        const float sg = even ? 1.f : -1.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float ox = __shfl_xor_sync(wmask, P[i].x, 1), oy = __shfl_xor_sync(wmask, P[i].y, 1);
            const float x0 = even ? P[i].x : ox, x1 = even ? P[i].y : oy, x2 = even ? ox : P[i].x, x3 = even ? oy : P[i].y;
            const float sd = __fmaf_rn(x1, sg, x0);                                   // x0 + x1 (even) or x0 - x1 (odd)
            const float rx = __fmaf_rn(x3, -sg, __fadd_rn(sd, x2));                   // (sd + x2) - x3   or (sd + x2) + x3
            const float ry = __fadd_rn(__fmaf_rn(even ? x2 : sd, -1.f, even ? sd : x2), x3);   // (sd - x2) + x3 or (-sd + x2) + x3
            P[i] = make_float2(__fmul_rn(0.5f, rx), __fmul_rn(0.5f, ry));
        }
    }
    // round to half; the row maximum is over the rounded values (the NaN-propagating form flags threads that hold one)
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        P[i] = __half22float2(__floats2half2_rn(P[i].x, P[i].y));
        amax = max3_abs_nan(amax, P[i].x, P[i].y);
    }
    const bool has_nan = amax != amax;
    if (has_nan) {
        amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fmaxf(fabsf(P[i].x), fabsf(P[i].y)));
    }
    if ((tpr & 7) == 0) {
        amax = fmaxf(amax, __shfl_xor_sync(wmask, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(wmask, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(wmask, amax, 4));
        if (t8 == 0) atomicMax(amax_s + rloc, __float_as_uint(amax));
    } else {
        atomicMax(amax_s + rloc, __float_as_uint(amax));
    }
    __syncthreads();
    const float mx = __uint_as_float(amax_s[rloc]);
    const float scale = __fdiv_rn(fmaxf(mx, 1e-30f), 127.f);
    if (live && tin == 0) scales[m] = scale;
    const float sh16 = rnd<half>(scale);
    const float st = sh16 > 0.f ? sh16 : scale;          // a scale below half's range divides in float
    const bool fast = sh16 > 0.f && mx <= 65504.f && !has_nan;
    uint32_t c16[16];
    if (fast) {
        const float rcp = __frcp_rn(st);
        const float2 rcp2 = make_float2(rcp, rcp), nst2 = make_float2(-st, -st), magic = make_float2(12582912.f, 12582912.f);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float2 q0 = __fmul2_rn(P[i], rcp2);
            const float2 t = __ffma2_rn(__ffma2_rn(q0, nst2, P[i]), rcp2, q0);
            const float2 th = __half22float2(__floats2half2_rn(t.x, t.y));
            const float2 u = __fadd2_rn(th, magic);
            const int n0 = (int)__float_as_uint(u.x) - 0x4B400000, n1 = (int)__float_as_uint(u.y) - 0x4B400000;
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(c16[i]) : "r"(n1), "r"(n0));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int qx = clamp_rint_i8(rnd<half>(__fdiv_rn(P[i].x, st)), -128.f), qy = clamp_rint_i8(rnd<half>(__fdiv_rn(P[i].y, st)), -128.f);
            c16[i] = (uint32_t)(qx & 0xff) | ((uint32_t)(qy & 0xff) << 8);
        }
    }
    int8_t* qr = q + m * (int64_t)K + tin * 32;
    if (ROT == 256) {
        uint16_t* cb = reinterpret_cast<uint16_t*>(tbuf);
        const uint32_t order = tsw ? 0x3201u : 0x3210u;
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) cb[t8 + 8 * rr] = (uint16_t)__byte_perm(c16[rr], 0u, order);
        __syncwarp(wmask);
        const uint4 lo = reinterpret_cast<const uint4*>(tbuf)[2 * t8], hi = reinterpret_cast<const uint4*>(tbuf)[2 * t8 + 1];
        if (live) {
            reinterpret_cast<uint4*>(qr)[0] = lo;
            reinterpret_cast<uint4*>(qr)[1] = hi;
        }
    } else if (live) {
        uint32_t w[8];
        if (ROT == 64) {      // c16[i] = codes of elements (i, i + 16)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t a = __byte_perm(c16[4 * j], c16[4 * j + 1], 0x5140), b = __byte_perm(c16[4 * j + 2], c16[4 * j + 3], 0x5140);
                w[j] = __byte_perm(a, b, 0x5410);          // bytes: codes of elements 4j .. 4j+3
                w[4 + j] = __byte_perm(a, b, 0x7632);      // and of elements 16+4j .. 16+4j+3
            }
        } else {              // c16[i] = codes of elements (2i, 2i + 1)
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = (c16[2 * i] & 0xffffu) | (c16[2 * i + 1] << 16);
        }
        reinterpret_cast<uint4*>(qr)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(qr)[1] = make_uint4(w[4], w[5], w[6], w[7]);
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

// gpu_sd_quant_rows through the register kernel above; false when the shape is not one it takes (the caller falls back).
bool b200q::sd_quant_rows_fast(const void* x, int64_t x_stride, int8_t* q, float* scales, int M, int K, int rotate, cudaStream_t st,
                               int* rc) {
    if (K % 32 || K > 16384 || (rotate == 64 && K % 64) || (rotate == 256 && K % 256) || (rotate != 0 && rotate != 64 && rotate != 256))
        return false;
    if ((((uintptr_t)x | (uintptr_t)q) & 15) || (x_stride & 7)) return false;
    const int tpr = K / 32;
    int rows = 256 / tpr;
    if (rows < 1) rows = 1;
    if (rows * tpr < 32) rows = (32 + tpr - 1) / tpr;
    const int threads = rows * tpr;
    const uint32_t off_amax = rotate == 256 ? (uint32_t)((threads + 31) / 32) * kWarpWords * 4 : 0;
    const size_t smem = off_amax + (size_t)rows * 4;
    const unsigned grid = (unsigned)((M + rows - 1) / rows);
    const half* xh = (const half*)x;
    *rc = 0;
    if (rotate == 256) {
        static std::atomic<uint64_t> configured{0};
        int dev = 0;
        cudaGetDevice(&dev);
        const uint64_t bit = 1ull << (dev & 63);
        if (smem > 48 * 1024 && !(configured.load(std::memory_order_acquire) & bit)) {
            const cudaError_t e = cudaFuncSetAttribute(sd_quant_fast_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            if (e != cudaSuccess) { *rc = (int)e; return true; }
            configured.fetch_or(bit, std::memory_order_release);
        }
        sd_quant_fast_kernel<256><<<grid, threads, smem, st>>>(xh, x_stride, q, scales, M, K, tpr, rows, off_amax);
    } else if (rotate == 64) {
        sd_quant_fast_kernel<64><<<grid, threads, smem, st>>>(xh, x_stride, q, scales, M, K, tpr, rows, off_amax);
    } else {
        sd_quant_fast_kernel<0><<<grid, threads, smem, st>>>(xh, x_stride, q, scales, M, K, tpr, rows, off_amax);
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) *rc = (int)e;
    return true;
}

// Reads and clears the quantizer's status word (a staging wait that ran out); used by gpu_kernels_status.
int b200q::quant_status_read_clear(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_quant_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_quant_status, &zero, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    *out = v;
    return 0;
}

// Device address of the bf16 -> bf16 table of a GEMM-epilogue activation (epilogue.cuh's Act codes), built on first use
// like the quantizer's own: the epilogue's out(act(out(v))) on bf16 outputs is a function of 16 bits.
int b200q::act_lut_ptr(int act, cudaStream_t st, const uint16_t** out) {
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

int sm_count_of(int dev) {
    static int count[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    int& c = count[dev & 63];
    if (c == 0) cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev);
    return c;
}

// CTAs of one kernel instantiation that fit an SM at a given size: asked of the runtime once per (threads, smem).
struct OccCache {
    std::mutex mu;
    int threads[8] = {}, blocks[8] = {}, n = 0;
    size_t smem[8] = {};
};

template <typename T, int PRO, int MAXT>
int launch_cfg(QuantArgs& p, int threads, size_t smem, bool persistent, cudaStream_t st) {
    auto kern = quant_rows_kernel<T, PRO, MAXT>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024) {
        const uint64_t bit = 1ull << (dev & 63);
        if (!(configured.load(std::memory_order_acquire) & bit)) {
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return (int)e;
            configured.fetch_or(bit, std::memory_order_release);
        }
    }
    int grid = p.nblocks;
    if (persistent) {
        static OccCache occ;
        int per_sm = 0;
        {
            std::lock_guard<std::mutex> lk(occ.mu);
            for (int i = 0; i < occ.n; ++i)
                if (occ.threads[i] == threads && occ.smem[i] == smem) per_sm = occ.blocks[i];
            if (!per_sm) {
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem) != cudaSuccess || per_sm < 1) {
                    (void)cudaGetLastError();
                    per_sm = 1;
                }
                const int slot = occ.n < 8 ? occ.n++ : 7;
                occ.threads[slot] = threads, occ.smem[slot] = smem, occ.blocks[slot] = per_sm;
            }
        }
        const int resident = per_sm * sm_count_of(dev);
        if (grid > resident) grid = resident;
    }
    kern<<<grid, threads, smem, st>>>(p);
    KCHECK();
    return 0;
}

constexpr size_t kMaxSmem = 227 * 1024;


template <typename T, int PRO>
int launch_quant(QuantArgs& p, cudaStream_t st) {
    p.tpr = p.K / 32;
    if (p.tpr > 1024) return -2;  // the reference's limit: K <= 32768 (csrc/kernels.cu:264)
    if (p.M <= 0) return 0;
    // 16-byte loads and bulk copies: rows must start 16-byte aligned, as the reference's load8 requires too
    const uintptr_t mis = (uintptr_t)p.x | (uintptr_t)(p.x_stride * sizeof(T)) |
                          (PRO == PRO_GATE ? (uintptr_t)p.g | (uintptr_t)(p.g_stride * sizeof(T)) : 0) |
                          (has_aux<PRO>() && PRO != PRO_GATE ? (uintptr_t)(p.up_offset * sizeof(T)) : 0) | (uintptr_t)p.q |
                          (uintptr_t)p.out_f | (uintptr_t)p.out_hi | (uintptr_t)p.out_lo;
    if (mis & 15) return -5;
    int lut = -1;
    if (sizeof(T) == 2 && (int64_t)p.M * p.K >= (1 << 20)) {
        lut = PRO == PRO_SILU || PRO == PRO_SWIGLU ? LUT_SILU : PRO == PRO_GELU ? LUT_GELU : PRO == PRO_GELU_TANH ? LUT_GELU_TANH
              : PRO == PRO_GATE ? LUT_SIGMOID : -1;
    }
    if (lut >= 0) {
        if (int rc = ensure_lut(lut, st)) return rc;
    }
    p.lut = lut;
    // CTA shape: whole rows, about 256 threads, at least one warp; any multiple of 8 threads up to 1024 works (the
    // last warp may be partial), so every K the reference accepts is served
    int rows = 256 / p.tpr;
    if (rows < 1) rows = 1;
    if (rows * p.tpr < 32) rows = (32 + p.tpr - 1) / p.tpr;
    p.rows_per_cta = rows;
    p.nblocks = (p.M + rows - 1) / rows;
    const int threads = rows * p.tpr;
    auto up = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
    size_t off = (size_t)((threads + 31) / 32) * kWarpWords * 4;
    p.off_amax = (uint32_t)off, off += (size_t)3 * rows * 4;
    p.off_norm = (uint32_t)off, off += is_norm<PRO>() ? (size_t)rows * norm_words(p.K) * 4 : 0;
    off = up(off, 16);
    off = up(off, 8);
    p.off_bar = (uint32_t)off, off += 8;
    off = up(off, 128);
    p.off_stage = (uint32_t)off;
    const size_t stage_bytes = (size_t)rows * p.K * sizeof(T) * (has_aux<PRO>() ? 2 : 1);
    // Measured on B200 (M = 4352, K = 12288, bf16): without the rotation, persistent CTAs with the next block's rows in
    // flight through the staging buffer win (49 against 54 us); with it the kernel is bound by its arithmetic and the
    // transposition, not by waiting for HBM, and one block per CTA with direct loads is as fast or faster (74 against 78).
    p.staged = !p.rotate && !is_norm<PRO>() && off + stage_bytes <= kMaxSmem;
    const size_t smem = p.staged ? off + stage_bytes : off;
    if (smem > kMaxSmem) return -2;
    if (threads > 512) return launch_cfg<T, PRO, 1024>(p, threads, smem, p.staged != 0, st);
    if (threads > 384) return launch_cfg<T, PRO, 512>(p, threads, smem, p.staged != 0, st);
    return launch_cfg<T, PRO, 384>(p, threads, smem, p.staged != 0, st);
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

// The same with the rotated rows written as two bf16 terms (hi + lo carries 16 significant bits of every value): the
// A operand of the weight-only int8 linear on the bf16 tensor-core kernel.
int b200q::rotate_rows_split(int prologue, const float* x, int64_t x_stride, int64_t up_offset, const float* norm_w, float eps,
                             void* hi, void* lo, int M, int K, cudaStream_t st) {
    if ((K % 256) != 0) return -1;
    QuantArgs p{x, x_stride, nullptr, 0, up_offset, nullptr, nullptr, nullptr, M, K, 1, 0, 0, 0, -1, nullptr, nullptr,
                norm_w, nullptr, eps, nullptr, nullptr};
    p.out_hi = reinterpret_cast<bf16*>(hi), p.out_lo = reinterpret_cast<bf16*>(lo);
    switch (prologue) {
        case PRO_PLAIN: return launch_quant<float, PRO_PLAIN>(p, st);
        case PRO_RMS: return launch_quant<float, PRO_RMS>(p, st);
        case PRO_SWIGLU: return launch_quant<float, PRO_SWIGLU>(p, st);
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

// ---- second pass after a rotating GEMM epilogue -------------------------------------------------------------------------
// gpu_int8_gemm_act_rot leaves the rows rotated and rounded to bf16, and per row N / 64 partial maxima of the unrounded
// rotated values (sign bit: a NaN among them), stored part-major [N / 64, M]. What is left of the quantizer is the row
// maximum, the scale and one pass over the row: 2 bytes read and 1 written per element. A CTA takes 8 consecutive rows
// (whose partial maxima are 32 contiguous bytes per part), `wpr` warps per row; a lane converts 16 consecutive values per
// step.
namespace {
constexpr int kRotRows = 8;
__global__ void __launch_bounds__(512) quant_rotated_kernel(const bf16* __restrict__ xr, const float* __restrict__ parts,
                                                            int8_t* __restrict__ q, float* __restrict__ scales, int M, int K,
                                                            int P, int wpr) {
    __shared__ unsigned s_amax[kRotRows], s_flag[kRotRows];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rloc = warp / wpr, seg = warp - rloc * wpr;
    const int64_t m0 = (int64_t)blockIdx.x * kRotRows, m = m0 + rloc;
    const bool live = m < M;
    const int per = K / wpr;
    const bf16* src = xr + m * (int64_t)K + (int64_t)seg * per;
    int8_t* dst = q + m * (int64_t)K + (int64_t)seg * per;
    if (threadIdx.x < kRotRows) s_amax[threadIdx.x] = 0u, s_flag[threadIdx.x] = 0u;
    // the first two steps' values are requested before the row's maximum is known: the partial maxima and the rows then
    // arrive together instead of one after the other
    uint4 a0, b0, a1, b1;
    a0 = b0 = a1 = b1 = make_uint4(0, 0, 0, 0);
    const int e0 = lane * 16;
    if (live && e0 < per) a0 = __ldg(reinterpret_cast<const uint4*>(src + e0)), b0 = __ldg(reinterpret_cast<const uint4*>(src + e0 + 8));
    if (live && e0 + 512 < per) a1 = __ldg(reinterpret_cast<const uint4*>(src + e0 + 512)), b1 = __ldg(reinterpret_cast<const uint4*>(src + e0 + 520));
    __syncthreads();
    // the 8 rows' partial maxima, 8 consecutive floats per part; non-negative floats order as integers
    for (int i = threadIdx.x; i < P * kRotRows; i += blockDim.x) {
        const int r = i & (kRotRows - 1);
        if (m0 + r < M) {
            const uint32_t u = __float_as_uint(__ldg(parts + (int64_t)(i >> 3) * M + m0 + r));
            atomicMax(&s_amax[r], u & 0x7fffffffu);
            if (u & 0x80000000u) s_flag[r] = 1u;
        }
    }
    __syncthreads();
    if (!live) return;
    const float amax = __uint_as_float(s_amax[rloc]);
    const uint32_t flag = s_flag[rloc];
    const float scale = fmaxf(fminf(amax, finite_max<bf16>()) * (1.f / 127.f), 1.0e-30f);
    if (seg == 0 && lane == 0) scales[m] = scale;
    const float st = rnd<bf16>(scale);
    // rows holding an infinity or a NaN keep the IEEE division and the exact clamp
    const bool fast = amax <= FLT_MAX && flag == 0;
    const float rcp = fast ? __frcp_rn(st) : 0.f;
    auto convert = [&](const uint4 a, const uint4 b, int e) {
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t c[8];
        if (fast) {
#pragma unroll
            for (int i = 0; i < 8; ++i) c[i] = quant2_bf16_bits(w[i], rcp);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                c[i] = quant2<bf16>(make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u)), st, 0.f, false);
        }
        *reinterpret_cast<uint4*>(dst + e) = make_uint4((c[0] & 0xffffu) | (c[1] << 16), (c[2] & 0xffffu) | (c[3] << 16),
                                                        (c[4] & 0xffffu) | (c[5] << 16), (c[6] & 0xffffu) | (c[7] << 16));
    };
    // two steps in flight: a step's values are replaced by those of the step after next before it is converted
#pragma unroll 1
    for (int e = e0; e < per; e += 1024) {
        uint4 a = a0, b = b0;
        if (e + 1024 < per) a0 = __ldg(reinterpret_cast<const uint4*>(src + e + 1024)), b0 = __ldg(reinterpret_cast<const uint4*>(src + e + 1032));
        convert(a, b, e);
        if (e + 512 < per) {
            a = a1, b = b1;
            if (e + 1536 < per) a1 = __ldg(reinterpret_cast<const uint4*>(src + e + 1536)), b1 = __ldg(reinterpret_cast<const uint4*>(src + e + 1544));
            convert(a, b, e + 512);
        }
    }
}
}  // namespace

// New: the quantizer's second pass on rows a rotating GEMM epilogue left (gpu_int8_gemm_act_rot): xr [M, K] bf16, rotated;
// amax_part [K / 64, M]; q [M, K] int8 and scales [M] as gpu_quant_rows(prologue = that activation, rotate = 1) gives them
// on the plain GEMM's output. K % 256 == 0 (-1); xr and q 16-byte aligned (-5).
GPU_API int gpu_quant_rows_rotated(const void* xr, const float* amax_part, int8_t* q, float* scales, int M, int K, void* stream) {
    if (K <= 0 || (K % 256) != 0) return -1;
    if (M <= 0) return 0;
    if ((((uintptr_t)xr | (uintptr_t)q) & 15) != 0) return -5;
    // enough warps for every SM to have many loads in flight: two warps share a long row
    const int wpr = K >= 4096 ? 2 : 1;
    const unsigned grid = (unsigned)((M + kRotRows - 1) / kRotRows);
    quant_rotated_kernel<<<grid, kRotRows * wpr * 32, 0, (cudaStream_t)stream>>>(reinterpret_cast<const bf16*>(xr), amax_part, q,
                                                                                 scales, M, K, K / 64, wpr);
    KCHECK();
    return 0;
}
