// int8 x int8 -> int32 GEMM with the fused dequant epilogue, for sm_100a.
//
//   D[m,n] = out( (sum_k A[m,k] * W[n,k]) * xs[m] * ws[n] + bias[n] )                       gpu_int8_gemm
//   D[m,n] = out( resid[m,n] + rscale[n] * out( acc * xs[m] * ws[n] + bias[n] ) )            gpu_int8_gemm_residual
//   D[m,n] = out( act( out( acc * xs[m] * ws[n] + bias[n] ) ) )                              gpu_int8_gemm_act (new)
//
// These are the entry points the reference exports from csrc/gemm.cu:123-140 over its CUTLASS 2.x
// mma.sync kernels (csrc/vendor/cutlass_gemm_int8.cu); the rounding points are those of its epilogue
// visitor trees (:84-95 plain, :143-161 residual), with the two multiply-adds fused as nvcc fuses them there.
//
// A cluster of two CTAs (two SMs) computes a 256 x bn tile with tcgen05.mma cta_group::2, kind::i8:
//   - each CTA stages its own 128 rows of A and its own bn/2 rows of W, 128 bytes of K per TMA box with the
//     128-byte swizzle (cp.async.bulk.tensor, never multicast), in a ring of shared-memory stages of one or two
//     boxes per operand; the byte counts of both CTAs are credited to the leader's "full" mbarrier
//   - warp 1 of the leader CTA (cluster rank 0) issues the MMAs for both SMs (M = 256, N = bn, K = 32 each) into
//     one of two tensor-memory accumulators; a commit releases a stage in both CTAs, another hands the finished
//     accumulator to both epilogues
//   - warps 2-9 of each CTA drain that CTA's 128 accumulator rows (two warps per TMEM lane quarter, splitting the
//     32-column chunks), apply scales / bias / activation or residual, round, and write through shared memory with
//     TMA stores (full-line writes; a direct-store path serves outputs that TMA cannot address)
//   - the persistent grid walks the tiles round-robin; bn is chosen per shape so the last round is not mostly idle
// Every wait is bounded; a wait that runs out records a code in g_kernel_status and the CTA pair unwinds.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cuda.h>
#include <cuda_fp8.h>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "epilogue.cuh"
#include "w6_decode.cuh"

__device__ int g_kernel_status = 0;

namespace {

constexpr int BM = 128;        // rows of A per CTA = TMEM lanes
constexpr int BK = 128;        // int8 elements (= bytes) of K per TMA box: one 128-byte swizzle row
constexpr int UMMA_K = 32;     // K of one tcgen05.mma kind::i8
constexpr int kThreads = 320;  // warp 0 producer, warp 1 MMA, warps 2-9 epilogue
constexpr int kEpiWarps = 8;
constexpr int64_t kResidentOperandBytes = 32ll << 20;   // an A this small stays in L2 while W and D stream past it
constexpr double kSmallProblemOps = 2.0e9;           // below this many int8 operations a GEMM takes the one-CTA-per-tile kernel
constexpr int kRotEpiWarps = 8;                      // epilogue warps of the rotating epilogue (two per tensor-memory lane quarter)
constexpr int kRotThreads = 64 + 32 * kRotEpiWarps;
constexpr int kMaxStages = 8;
constexpr int kSmemBytes = 232448;            // the per-CTA maximum (227 KB)
// Epilogue staging, 32 KB. 4-byte outputs: per warp 32 rows x 128 B. 2-byte outputs: per warp a 2 KB chunk buffer (32 rows x
// 64 B), then per warp the staged per-column vectors (ws | bias [| rscale], 128 floats each), and, for the activation
// epilogue, the shared-memory part of the activation table behind them (16 + 8 + 8 KB).
constexpr int kStagingBytes = kEpiWarps * 4096;
constexpr int kVecOffset = kEpiWarps * 2048;                 // 2-byte outputs: vectors start behind the chunk buffers
constexpr int kTailBytes = 512;               // barriers, tensor-memory pointer, abort flag, the rotating epilogue's flags

struct GemmParams {
    const float* xs;     // [M]
    const float* ws;     // [N]
    const void* bias;    // [N] out dtype, nullable
    const void* rscale;  // [N] out dtype (residual form)
    const void* resid;   // [M,N] out dtype (residual form), may alias D
    void* D;             // [M,N] out dtype, or int32 for EPI_ACC
    int M, N, K;
    int tiles_m, tiles_n, num_tiles, k_iters;
    int group_m;         // row tiles per band of the tile order (0 = the default of 8)
    int act;
    int vec_ok;          // per-column vectors and rows of D / resid can be read and written 16 bytes at a time
    int tma_store;       // D is written through shared memory with TMA stores
    int bn;              // columns per tile (multiple of 32, <= 256); each CTA of the pair stages bn/2 rows of W
    int stages;          // shared-memory ring depth
    int ksub;            // 128-byte K boxes per stage (1 or 2): one barrier round trip per 4 or 8 MMAs
    // Split tail: when the last round would hold only a few tiles, those tiles are cut along K into `splits` work items
    // each, so that round runs on every cluster; partial int32 accumulators meet in `scratch`.
    int whole_tiles;     // tiles computed in one piece (work items [0, whole_tiles))
    int splits;          // K slices per split tile (>= 2), or 0: work items [whole_tiles, whole_tiles + rem * splits)
    int kps;             // stages per K slice
    int num_items;       // whole_tiles + split tiles * splits
    int* scratch;        // counters [slot][2][4][8], zero between launches
    int* partials;       // [slot][2][4][8][32 values][32 lanes] int32 sums, zero between launches
    uint32_t idesc;      // instruction descriptor for M = 256, N = bn
    const uint16_t* act_lut;   // EPI_ACT with bf16 outputs: bf16(act(x)) for every bf16 x (a tanhf or erff per element
                               // made the epilogue, not the tensor core, the limit: 836 against 2740 TOPS), or null
    float* amax_part;          // EPI_ACT_ROT: [N / 64, M] partial row maxima of |rotated value| (four per tile, see the
                               // epilogue), sign bit set when the part held a NaN
};

// Tile order: bands of `group_m` row tiles, column tile fastest-varying across the band's rows, so that the clusters
// running at one time share a few A row-panels and W column-panels in L2. Eight rows per band balance the two operands
// (74 tiles at a time make about a square); the host side picks taller bands when the band's rows of A can stay in L2
// and W is too large to (up-projection M = 4352: one band, 109.7 against 113.3 us; 6144 x 5120 x 15360: 297 against 311).
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn, int group_m = 8) {
    const int per_group = group_m * tiles_n;
    const int group = t / per_group;
    const int first_m = group * group_m;
    const int gsize = min(group_m, tiles_m - first_m);
    const int r = t - group * per_group;
    tm = first_m + r % gsize;
    tn = r / gsize;
}

// Work item -> tile, K range (in stages) and, for a slice of a split tile, its slot in the scratch.
enum ItemKind { ITEM_WHOLE = 0, ITEM_SLICE = 1 };
struct WorkItem { int tile, k0, kn, kind, slot; };
__device__ __forceinline__ WorkItem decode_item(const GemmParams& p, int w) {
    if (w < p.whole_tiles) return {w, 0, p.k_iters, ITEM_WHOLE, 0};
    const int j = w - p.whole_tiles;
    const int slot = j / p.splits, sidx = j - slot * p.splits;
    const int k0 = sidx * p.kps;
    return {p.whole_tiles + slot, k0, min(p.kps, p.k_iters - k0), ITEM_SLICE, slot};
}
constexpr int kCountersPerSlot = 2 * 4 * 8;   // CTA of the pair x TMEM lane quarter x 32-column chunk

template <typename OutT> __device__ __forceinline__ uint4 pack8(const float (&y)[8]);
template <> __device__ __forceinline__ uint4 pack8<bf16>(const float (&y)[8]) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
    return *reinterpret_cast<uint4*>(h);
}
template <> __device__ __forceinline__ uint4 pack8<half>(const float (&y)[8]) {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
    return *reinterpret_cast<uint4*>(h);
}
template <typename OutT> __device__ __forceinline__ void load8(const OutT* p, float (&y)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&y)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    y[0] = a.x, y[1] = a.y, y[2] = a.z, y[3] = a.w, y[4] = b.x, y[5] = b.y, y[6] = b.z, y[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float (&y)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        y[2 * i] = f.x, y[2 * i + 1] = f.y;
    }
}
template <> __device__ __forceinline__ void load8<half>(const half* p, float (&y)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        y[2 * i] = f.x, y[2 * i + 1] = f.y;
    }
}

// 8 two-byte values held in a register quad -> floats (no address is taken: the quad stays in registers)
template <typename OutT> __device__ __forceinline__ void unpack8(const uint4 u, float (&y)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (std::is_same<OutT, bf16>::value) {
            y[2 * i] = __uint_as_float(w[i] << 16), y[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else if constexpr (std::is_same<OutT, half>::value) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            y[2 * i] = f.x, y[2 * i + 1] = f.y;
        } else {
            y[2 * i] = 0.f, y[2 * i + 1] = 0.f;
        }
    }
}

// The epilogue arithmetic on 8 consecutive columns of one row (accumulators r[0..7] -> y[0..7], not yet rounded
// to the output type for the last step; the store rounds).
//   t0 = float(acc) * xs;  v = out(fma(t0, ws, bias));  RESID: fma(v, rscale, resid);  ACT: act(v)
// `vs`, when set, points at this warp's staged per-column vectors for these 8 columns in shared memory
// (ws at vs[0..], bias at vs[VS..], rscale at vs[2 VS..], all as f32, zero beyond N; VS = columns a warp stages).
// The part of the 65536-entry activation table an epilogue keeps in shared memory: bf16 bit patterns of 2^-11 <= |x| < 32
// (16 exponents x 128 significands), positive half first; anything else is read from the whole table in global memory
// (a warp does that for a group of eight columns as soon as one of its 32 rows needs it, so the window sits where
// pre-activations of a normalised network fall: with a standard deviation of 0.5 to 5, one value in 1000 to 10000 lies
// below it and none above; a window reaching down to 2^-12 but only up to 16 cost the rotating epilogue 176 instead of 142 us
// once a residual stream had drifted to a standard deviation near 5).
// Inside a half the entry of pattern b sits at b & 0x7ff (the window 0x3A00..0x41FF wraps once), so the index needs no
// subtraction: (b & 0x7ff) | (sign << 11).
constexpr uint32_t kActLutLo = 0x3A00u, kActLutHalf = 16u * 128u;
constexpr float kActLutMinAbs = 0.00048828125f, kActLutMaxAbs = 31.875f;   // 2^-11; the largest bf16 below 32
__host__ __device__ constexpr uint32_t act_lut_pattern(uint32_t i) {   // bf16 pattern whose entry sits at index i of the shared part
    return ((i & 0x800u) << 4) | ((i & 0x7ffu) >= (kActLutLo & 0x7ffu) ? 0x3800u : 0x4000u) | (i & 0x7ffu);
}
__device__ __forceinline__ uint32_t act_lut_index(uint32_t b) { return (b & 0x7ffu) | ((b >> 4) & 0x800u); }
constexpr int kActLutBytes = 2 * (int)kActLutHalf * 2;

// Accumulator word -> float: int32 sums of the int8 kernel (KIND 0), or the f32 sums of the bf16 kernel (KIND 1) as they are.
template <int KIND> __device__ __forceinline__ float acc_f(uint32_t r) {
    return KIND == 0 ? __int2float_rn((int)r) : __uint_as_float(r);
}

template <typename OutT, int EPI, int VS = 128, int KIND = 0>
__device__ __forceinline__ void epilogue8(const GemmParams& p, const uint32_t* r, int row, int col, float xs_r, bool vec,
                                          float (&y)[8], const float* vs = nullptr, const uint16_t* lut_sm = nullptr,
                                          bool have_resid8 = false, const uint4 resid8 = uint4{0, 0, 0, 0}) {
    float w8[8], b8[8], rs8[8], rr[8];
    const OutT* rsd = reinterpret_cast<const OutT*>(p.resid) + (int64_t)row * p.N + col;
    if (vs) {
        load8<float>(vs, w8);            // every lane reads the same words: broadcasts
        load8<float>(vs + VS, b8);
        if (EPI == EPI_RESID) {
            load8<float>(vs + 2 * VS, rs8);
            if (have_resid8) unpack8<OutT>(resid8, rr);      // fetched by the caller, 8 two-byte values
            else if (vec) load8<OutT>(rsd, rr);
            else {
#pragma unroll
                for (int e = 0; e < 8; ++e) rr[e] = col + e < p.N ? to_f<OutT>(rsd[e]) : 0.f;
            }
        }
    } else if (vec) {
        // every lane reads the same addresses of the per-column vectors: one broadcast per load
        load8<float>(p.ws + col, w8);
        if (p.bias) load8<OutT>(reinterpret_cast<const OutT*>(p.bias) + col, b8);
        if (EPI == EPI_RESID) {
            if (p.rscale) load8<OutT>(reinterpret_cast<const OutT*>(p.rscale) + col, rs8);
            else {
#pragma unroll
                for (int e = 0; e < 8; ++e) rs8[e] = 1.f;
            }
            load8<OutT>(rsd, rr);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int n = col + e;
            const bool in = n < p.N;
            w8[e] = in ? p.ws[n] : 0.f;
            if (p.bias) b8[e] = in ? to_f<OutT>(reinterpret_cast<const OutT*>(p.bias)[n]) : 0.f;
            if (EPI == EPI_RESID) {
                rs8[e] = !in ? 0.f : p.rscale ? to_f<OutT>(reinterpret_cast<const OutT*>(p.rscale)[n]) : 1.f;
                rr[e] = in ? to_f<OutT>(rsd[e]) : 0.f;
            }
        }
    }
    if (!vs && !p.bias) {
#pragma unroll
        for (int e = 0; e < 8; ++e) b8[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float t0 = __fmul_rn(acc_f<KIND>(r[e]), xs_r);
        float v = rnd<OutT>(__fmaf_rn(t0, w8[e], b8[e]));
        if (EPI == EPI_RESID) v = __fmaf_rn(v, rs8[e], rr[e]);
        else if (EPI == EPI_ACT_LUT) {
            // bf16(act(v)) from the table: its hot part sits in shared memory, the rest is read from global memory
            // (a predicated load; the shared-memory index is masked into range either way)
            const uint32_t bits = __float_as_uint(v) >> 16;
            uint32_t t = lut_sm[act_lut_index(bits)];                                   // sign bit 15 -> the table's second half
            if (((bits & 0x7fffu) - kActLutLo) >= kActLutHalf) t = __ldg(p.act_lut + bits);
            v = __uint_as_float(t << 16);
        } else if (EPI == EPI_ACT) {
            v = p.act == ACT_GELU_TANH ? gelu_tanh_f(v) : p.act == ACT_SILU ? silu_f(v) : gelu_f(v);
        }
        y[e] = v;
    }
}

// The table-driven activation epilogue on 8 consecutive columns of one row, for bf16 outputs through the staged path:
// y = bf16(fma(float(acc) * xs, ws, bias)) is formed two at a time (one packed conversion), its 16 bits index the table
// (hot part in shared memory, sign in the index's top bit), and the table's 16-bit entries are the output as they are:
// no conversion back and forth. Values outside the shared-memory part (checked once per 8) are read from the whole table.
// Out of line on purpose: inlined, its eight loads were issued (predicated off) by every group of eight and cost the
// epilogue a tenth of its instructions.
__device__ __noinline__ uint4 act_lut_whole8(const uint16_t* __restrict__ lut, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
    const uint32_t w[4] = {w0, w1, w2, w3};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = (uint32_t)__ldg(lut + (w[i] & 0xffffu)) | ((uint32_t)__ldg(lut + (w[i] >> 16)) << 16);
    return make_uint4(o[0], o[1], o[2], o[3]);
}
// t[e] = table entry (16 bits) for column e. Returns false when some entry came from the whole table (values outside the
// shared-memory part: the caller may want to look at their size).
template <int VS>
__device__ __forceinline__ bool epilogue8_lut_bits(const GemmParams& p, const uint32_t* r, float xs_r, const float* vs,
                                                   const uint16_t* lut_sm, uint32_t (&t)[8]) {
    float w8[8], b8[8], v[8];
    load8<float>(vs, w8);
    load8<float>(vs + VS, b8);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[e]), xs_r), w8[e], b8[e]);
    // inside the shared-memory part when 2^-11 <= |v| < 31.875 for all eight (rounding to bf16 then stays below 32); a NaN
    // fails the comparison
    float lo = fabsf(v[0]), hi = lo;
#pragma unroll
    for (int e = 1; e < 7; e += 2) {
        asm("min.f32 %0, %1, %2, %3;" : "=f"(lo) : "f"(lo), "f"(fabsf(v[e])), "f"(fabsf(v[e + 1])));
        asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(hi) : "f"(hi), "f"(fabsf(v[e])), "f"(fabsf(v[e + 1])));
    }
    lo = fminf(lo, fabsf(v[7]));
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(hi) : "f"(hi), "f"(fabsf(v[7])));
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
        t[2 * i] = lut_sm[act_lut_index(w[i])];
        t[2 * i + 1] = lut_sm[act_lut_index(w[i] >> 16)];
    }
    const bool inside = lo >= kActLutMinAbs && hi < kActLutMaxAbs;
    if (__all_sync(0xffffffffu, inside)) return true;
    const uint4 o = act_lut_whole8(p.act_lut, w[0], w[1], w[2], w[3]);
    t[0] = o.x & 0xffffu, t[1] = o.x >> 16, t[2] = o.y & 0xffffu, t[3] = o.y >> 16;
    t[4] = o.z & 0xffffu, t[5] = o.z >> 16, t[6] = o.w & 0xffffu, t[7] = o.w >> 16;
    return false;
}
template <int VS>
__device__ __forceinline__ uint4 epilogue8_lut(const GemmParams& p, const uint32_t* r, float xs_r, const float* vs,
                                               const uint16_t* lut_sm) {
    uint32_t t[8];
    epilogue8_lut_bits<VS>(p, r, xs_r, vs, lut_sm, t);
    return make_uint4(t[0] | (t[1] << 16), t[2] | (t[3] << 16), t[4] | (t[5] << 16), t[6] | (t[7] << 16));
}

// Radix-4 butterfly of the regular Hadamard block on f32 bit patterns, outputs in the reference's association
// (csrc/common.cuh:99-126): r0 = .5*(((x0+x1)+x2)-x3)  r1 = .5*(((x0+x1)-x2)+x3)  r2 = .5*(((x0-x1)+x2)+x3)
// r3 = .5*(((-x0+x1)+x2)+x3); -x0+x1 is the exact negation of x0-x1.
__device__ __forceinline__ void h4u(uint32_t& u0, uint32_t& u1, uint32_t& u2, uint32_t& u3) {
    const float x0 = __uint_as_float(u0), x1 = __uint_as_float(u1), x2 = __uint_as_float(u2), x3 = __uint_as_float(u3);
    const float s = __fadd_rn(x0, x1), d = __fsub_rn(x0, x1);
    u0 = __float_as_uint(__fmul_rn(0.5f, __fsub_rn(__fadd_rn(s, x2), x3)));
    u1 = __float_as_uint(__fmul_rn(0.5f, __fadd_rn(__fsub_rn(s, x2), x3)));
    u2 = __float_as_uint(__fmul_rn(0.5f, __fadd_rn(__fadd_rn(d, x2), x3)));
    u3 = __float_as_uint(__fmul_rn(0.5f, __fadd_rn(__fsub_rn(x2, d), x3)));
}
// The same without the halving. With inputs scaled by a power of two instead, every intermediate is the reference's times
// a power of two: rounding commutes with such a scaling as long as nothing overflows (the caller bounds the inputs) and
// nothing is rounded in the subnormal range (sums of bf16 values are multiples of 2^-133, and so are their sixteenths' sums
// of 2^-137: subnormal results are exact).
__device__ __forceinline__ void h4n(uint32_t& u0, uint32_t& u1, uint32_t& u2, uint32_t& u3) {
    const float x0 = __uint_as_float(u0), x1 = __uint_as_float(u1), x2 = __uint_as_float(u2), x3 = __uint_as_float(u3);
    const float s = __fadd_rn(x0, x1), d = __fsub_rn(x0, x1);
    u0 = __float_as_uint(__fsub_rn(__fadd_rn(s, x2), x3));
    u1 = __float_as_uint(__fadd_rn(__fsub_rn(s, x2), x3));
    u2 = __float_as_uint(__fadd_rn(__fadd_rn(d, x2), x3));
    u3 = __float_as_uint(__fadd_rn(__fsub_rn(x2, d), x3));
}
// Stages of strides 1, 4 and 16 over 64 values held as two halves of 32
template <bool HALVE>
__device__ __forceinline__ void three_stages64(uint32_t (&ra)[32], uint32_t (&rb)[32]) {
    auto bf = [](uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
        if (HALVE) h4u(a, b, c, d);
        else h4n(a, b, c, d);
    };
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        bf(ra[i], ra[i + 1], ra[i + 2], ra[i + 3]);
        bf(rb[i], rb[i + 1], rb[i + 2], rb[i + 3]);
    }
#pragma unroll
    for (int b = 0; b < 32; b += 16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            bf(ra[b + i], ra[b + i + 4], ra[b + i + 8], ra[b + i + 12]);
            bf(rb[b + i], rb[b + i + 4], rb[b + i + 8], rb[b + i + 12]);
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) bf(ra[i], ra[i + 16], rb[i], rb[i + 16]);
}
// max(m, |a|, |b|) that is NaN as soon as one input is
__device__ __forceinline__ float max3_abs_nan_u(float m, uint32_t a, uint32_t b) {
    float o;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(o) : "f"(m), "f"(fabsf(__uint_as_float(a))), "f"(fabsf(__uint_as_float(b))));
    return o;
}

// One 32-column chunk of one accumulator row, written straight to global memory (the path for outputs whose row
// pitch or base TMA cannot address, and for ragged N).
template <typename OutT, int EPI, int KIND = 0>
__device__ __forceinline__ void chunk_direct(const GemmParams& p, const uint32_t (&r)[32], int row, int col0, float xs_r) {
    if (EPI == EPI_ACC) {
        int32_t* d = reinterpret_cast<int32_t*>(p.D) + (int64_t)row * p.N + col0;
        if (p.vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(d + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) d[j] = (int32_t)r[j];
        }
        return;
    }
    OutT* d = reinterpret_cast<OutT*>(p.D) + (int64_t)row * p.N + col0;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        if (col0 + j >= p.N) break;
        const bool vec = p.vec_ok && col0 + j + 8 <= p.N;
        float y[8];
        epilogue8<OutT, EPI, 128, KIND>(p, r + j, row, col0 + j, xs_r, vec, y);
        if (vec) {
            if constexpr (sizeof(OutT) == 2) {
                *reinterpret_cast<uint4*>(d + j) = pack8<OutT>(y);
            } else {
                reinterpret_cast<float4*>(d + j)[0] = make_float4(y[0], y[1], y[2], y[3]);
                reinterpret_cast<float4*>(d + j)[1] = make_float4(y[4], y[5], y[6], y[7]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (col0 + j + e < p.N) d[j + e] = from_f<OutT>(y[e]);
        }
    }
}

// One 32-column chunk of the warp's 32 rows, staged in shared memory in the layout a TMA store with the 64-byte
// (2-byte outputs) or 128-byte (4-byte outputs) swizzle expects: row r at r * pitch, its 16-byte piece j at
// piece j ^ f(r). Eight consecutive lanes then hit eight different bank groups.
// 2-byte outputs: the chunk's 32 values of this lane's row, computed and packed (no shared-memory traffic yet)
template <typename OutT, int EPI, int VS = 128, int KIND = 0>
__device__ __forceinline__ void chunk_compute16(const GemmParams& p, const uint32_t (&r)[32], int row, int col0, float xs_r,
                                                const float* vs, uint4 (&pk)[4], const uint16_t* lut_sm = nullptr) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if constexpr (EPI == EPI_ACT_LUT) {
            pk[j] = epilogue8_lut<VS>(p, r + 8 * j, xs_r, vs + 8 * j, lut_sm);
        } else {
            float y[8];
            epilogue8<OutT, EPI, VS, KIND>(p, r + 8 * j, row, col0 + 8 * j, xs_r, p.vec_ok && col0 + 8 * j + 8 <= p.N, y, vs + 8 * j, lut_sm);
            if constexpr (sizeof(OutT) == 2) pk[j] = pack8<OutT>(y);
        }
    }
}
// The residual form of the same with the residual's four 16-byte pieces of this row already fetched by the caller
template <typename OutT, int VS = 128, int KIND = 0>
__device__ __forceinline__ void chunk_compute16_resid(const GemmParams& p, const uint32_t (&r)[32], int row, int col0, float xs_r,
                                                      const float* vs, uint4 (&pk)[4], const uint4 (&rq)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float y[8];
        epilogue8<OutT, EPI_RESID, VS, KIND>(p, r + 8 * j, row, col0 + 8 * j, xs_r, true, y, vs + 8 * j, nullptr, true, rq[j]);
        if constexpr (sizeof(OutT) == 2) pk[j] = pack8<OutT>(y);
    }
}
__device__ __forceinline__ void chunk_write16(const uint4 (&pk)[4], uint8_t* stage, int lane) {
    uint8_t* rowp = stage + lane * 64;
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(rowp + ((j ^ sw) << 4)) = pk[j];
}

template <typename OutT, int EPI, int KIND = 0>
__device__ __forceinline__ void chunk_to_smem(const GemmParams& p, const uint32_t (&r)[32], int row, int col0, float xs_r,
                                              uint8_t* stage, int lane) {
    constexpr int kEsz = EPI == EPI_ACC ? 4 : (int)sizeof(OutT);
    if constexpr (kEsz == 2) {
        return;   // 2-byte outputs go through chunk_compute16 / chunk_write16
    } else {
        uint8_t* rowp = stage + lane * 128;
        const int sw = lane & 7;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float y[8];
            if (EPI == EPI_ACC) {
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = __uint_as_float(r[8 * j + e]);  // raw int32 bits
            } else {
                epilogue8<OutT, EPI, 128, KIND>(p, r + 8 * j, row, col0 + 8 * j, xs_r, p.vec_ok && col0 + 8 * j + 8 <= p.N, y);
            }
            *reinterpret_cast<float4*>(rowp + (((2 * j) ^ sw) << 4)) = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4*>(rowp + (((2 * j + 1) ^ sw) << 4)) = make_float4(y[4], y[5], y[6], y[7]);
        }
    }
}

// 2-D tiled TMA store, shared memory -> global; rows and columns beyond the tensor are clipped.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tmap), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// ---- the rotating epilogue (EPI_ACT_ROT) --------------------------------------------------------------------------------
// Activation, then the R256 rotation of the tile's 256 columns (one rotation group per row), written as bf16 with the
// row's maximum over this warp's share beside it: what the quantizer's second pass needs. Tile width 256, bf16 and whole
// tiles only (the host side sees to it). The two warps of a lane quarter split the work, and tensor memory is their
// scratch (the accumulator is rewritten in place, as f32). Warp h of the two:
//   1  columns [128 h, 128 h + 128) as two 64-column blocks: dequantize, activation from the table, the stages of strides
//      1, 4 and 16 (64 values in registers), back to tensor memory; barrier between the two warps;
//   2  the last stage (columns j, j + 64, j + 128, j + 192) for the offsets j in [32 h, 32 h + 32), sixteen at a time: row
//      maximum, rounding to bf16, and out through shared memory with TMA stores of 16-column boxes, two per fence.
// This epilogue, not the tensor core, bounds the kernel (builds with one part of it left out each: the tensor-memory stores,
// the staged stores and the butterflies cost about as much each, the table look-ups a third of that), and its warps wait
// for latency and instruction fetch, not for issue slots: the loops are kept rolled (fully unrolled, "no instruction" was
// the largest stall), and the next tile's per-column vectors and row scale are fetched a tile ahead. Plain 16-byte stores
// from the registers (a row per lane) were slower than the staged TMA stores, and so were sixteen warps instead of eight
// and a pass of its own for the table look-ups (eight columns a step through tensor memory).
__device__ __forceinline__ void rotate_block64(uint32_t (&a)[32], uint32_t (&b)[32], bool exact) {
    // Three stages (strides 1, 4, 16) of one 64-column block, left as half the reference's values: without the per-stage
    // halvings and one multiplication by 1/16 at the end, or, next to huge values (where the unhalved sums could overflow
    // although the reference's do not), exactly as the reference computes them, then halved (exact: see h4n).
    if (!exact) {
        three_stages64<false>(a, b);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            a[i] = __float_as_uint(__fmul_rn(__uint_as_float(a[i]), 0.0625f));
            b[i] = __float_as_uint(__fmul_rn(__uint_as_float(b[i]), 0.0625f));
        }
    } else {
        three_stages64<true>(a, b);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            a[i] = __float_as_uint(__fmul_rn(__uint_as_float(a[i]), 0.5f));
            b[i] = __float_as_uint(__fmul_rn(__uint_as_float(b[i]), 0.5f));
        }
    }
}

__device__ __forceinline__ void epilogue_rot(const GemmParams& p, const CUtensorMap* tmap_d16, uint8_t* staging, uint8_t* tail,
                                             uint32_t bar_tfull, uint32_t bar_tempty, uint32_t tmem_base, volatile int* abort_s,
                                             int rank, int cluster_id, int nclusters, int warp, int lane) {
    const int ew = warp - 2;
    const int quad = warp & 3;               // TMEM lane quarter this warp may read
    const int half = ew >> 2;
    uint8_t* my_stage = staging + ew * 2048;                                              // two buffers of 32 rows x 32 bytes
    const uint32_t my_stage_u32 = smem_u32(my_stage);
    float* my_vec = reinterpret_cast<float*>(staging + kVecOffset + ew * 1024);          // ws[128] | bias[128]
    const uint16_t* lut_sm = reinterpret_cast<const uint16_t*>(staging + kVecOffset + kEpiWarps * 1024);
    volatile int* pair_ok = reinterpret_cast<volatile int*>(tail + 176);                  // [tile parity][quarter][half]
    const bf16* bias = reinterpret_cast<const bf16*>(p.bias);
    int buf = 0;
    uint32_t tphase = 0;

    // this warp's columns of ws / bias and this lane's row scale, for the tile `w`
    float nx_ws[4], nx_b[4], nx_xs = 1.f;
    auto fetch = [&](int w) {
        int tm, tn;
        tile_coords(w, p.tiles_m, p.tiles_n, tm, tn, p.group_m ? p.group_m : 8);
        const int row = tm * (2 * BM) + rank * BM + quad * 32 + lane;
        nx_xs = p.xs ? __ldg(p.xs + (row < p.M ? row : p.M - 1)) : 1.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int n = tn * 256 + (4 * half + k) * 32 + lane;
            nx_ws[k] = __ldg(p.ws + n);
            nx_b[k] = bias ? __bfloat162float(bias[n]) : 0.f;
        }
    };
    if (cluster_id < p.num_items) fetch(cluster_id);

    for (int w = cluster_id; w < p.num_items; w += nclusters) {
        int tm, tn;
        tile_coords(w, p.tiles_m, p.tiles_n, tm, tn, p.group_m ? p.group_m : 8);
        const int n0 = tn * 256;
        const int row0 = tm * (2 * BM) + rank * BM + quad * 32;
        const int row = row0 + lane;
        const float xs_r = nx_xs;
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            my_vec[32 * k + lane] = nx_ws[k];
            my_vec[128 + 32 * k + lane] = nx_b[k];
        }
        __syncwarp();
        if (w + nclusters < p.num_items) fetch(w + nclusters);      // in flight while this tile is processed

        const bool got = mbar_wait_warp_relaxed(bar_tfull + 8 * buf, tphase, abort_s, ST_TIMEOUT_TMEM_FULL);
        tc_fence_after();
        const uint32_t taddr = tmem_base + buf * 256 + ((uint32_t)(quad * 32) << 16);
        bool big = false;   // a value of 2^120 or more (or an infinity, a NaN) among this warp's: exact halvings
        if (got) {
            const uint32_t ta = taddr + 128 * half;
            // A + B per 64-column block: dequantize, activation from the table, three stages, back to tensor memory
            // (loading the next half block ahead of its use through a third register set was slower: 1.23 against 1.21
            // times the plain kernel; so was keeping this warp's own half of every block in registers and sending only
            // the partner's half through tensor memory: 1.28, the last stage then has to be unrolled over its two steps)
#pragma unroll 1
            for (int blk = 0; blk < 2; ++blk) {
                uint32_t a[32], b[32];
                tmem_ld32(ta + 64 * blk, a);
                tmem_ld32(ta + 64 * blk + 32, b);
                tmem_ld_wait();
                bool wide = false;
                const float* vs = my_vec + 64 * blk;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t t[8];
                    if (!epilogue8_lut_bits<128>(p, a + 8 * j, xs_r, vs + 8 * j, lut_sm, t)) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) wide |= (t[e] & 0x7fffu) >= 0x7B80u;
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[8 * j + e] = t[e] << 16;
                    if (!epilogue8_lut_bits<128>(p, b + 8 * j, xs_r, vs + 32 + 8 * j, lut_sm, t)) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) wide |= (t[e] & 0x7fffu) >= 0x7B80u;
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) b[8 * j + e] = t[e] << 16;
                }
                const bool ex = __any_sync(0xffffffffu, wide);
                big |= ex;
                rotate_block64(a, b, ex);
                tmem_st32(ta + 64 * blk, a);
                tmem_st32(ta + 64 * blk + 32, b);
            }
            tmem_st_wait();
        }
        // The partner's blocks are needed next. A warp whose wait ran out still meets its partner here, and both leave
        // together: the decision is read from flags written before the barrier (two sets, by tile parity: a warp is at
        // most one barrier ahead of its partner).
        if (lane == 0) pair_ok[(buf * 4 + quad) * 2 + half] = got ? (big ? 3 : 1) : 0;
        tc_fence_before();
        named_bar_sync(1 + quad, 64);
        tc_fence_after();
        const int f0 = pair_ok[(buf * 4 + quad) * 2], f1 = pair_ok[(buf * 4 + quad) * 2 + 1];
        if (!f0 || !f1) break;
        const bool exact = ((f0 | f1) & 2) != 0;     // either warp met huge values: the last stage as the reference has it

        // C: the last stage, sixteen offsets a step
        const bool row_ok = row < p.M;
#pragma unroll 1
        for (int t = 0; t < 2; ++t) {
            const int j0 = 32 * half + 16 * t;
            uint32_t q[4][16];
#pragma unroll
            for (int k = 0; k < 4; ++k) tmem_ld16(taddr + 64 * k + j0, q[k]);
            tmem_ld_wait();
            if (t == 1) {
                // The accumulator is free as soon as both warps have read it. No cluster-scope release: nothing but tensor
                // memory, ordered by the tcgen05 fences, is handed over.
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(mapa_shared(bar_tempty + 8 * buf, 0));
            }
            if (!exact) {
#pragma unroll
                for (int i = 0; i < 16; ++i) h4n(q[0][i], q[1][i], q[2][i], q[3][i]);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) q[k][i] = __float_as_uint(__fmul_rn(__uint_as_float(q[k][i]), 2.f));
                    h4u(q[0][i], q[1][i], q[2][i], q[3][i]);
                }
            }
            float m = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
#pragma unroll
                for (int i = 0; i < 16; i += 2) m = max3_abs_nan_u(m, q[k][i], q[k][i + 1]);
            }
            bool has_nan = false;
            if (m != m) {   // the reference's fmaxf drops a NaN: the maximum again without it, and a flag
                has_nan = true;
                m = 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(__uint_as_float(q[k][i])));
                }
            }
            // part-major, so that a warp's 32 rows make one 128-byte store (row-major, the 4-byte stores of a warp went to
            // 32 different sectors, each of them written eight times over the launch: at 16896 rows, where the output
            // streams through L2, that made the kernel 1.6 times the plain one instead of 1.2)
            if (row_ok)
                p.amax_part[(int64_t)(4 * tn + 2 * half + t) * p.M + row] = has_nan ? __uint_as_float(__float_as_uint(m) | 0x80000000u) : m;
            // out through the two staging buffers, two 16-column pieces per fence and store group
#pragma unroll
            for (int kp = 0; kp < 4; kp += 2) {
                uint32_t o[2][8];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(q[kp + u][2 * i]), __uint_as_float(q[kp + u][2 * i + 1]));
                        o[u][i] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                }
                if (lane == 0) bulk_wait_read<0>();   // the previous group's stores have read both buffers
                __syncwarp();
                // 32-byte rows with the 32-byte swizzle (the 16-byte half is flipped in every other group of four rows):
                // without it rows r and r + 4 meet in the same banks
                const int flip = ((lane >> 2) & 1) << 4;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    uint8_t* rowp = my_stage + u * 1024 + lane * 32;
                    *reinterpret_cast<uint4*>(rowp + flip) = make_uint4(o[u][0], o[u][1], o[u][2], o[u][3]);
                    *reinterpret_cast<uint4*>(rowp + (16 ^ flip)) = make_uint4(o[u][4], o[u][5], o[u][6], o[u][7]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(tmap_d16, my_stage_u32, n0 + 64 * kp + j0, row0);
                    tma_store_2d(tmap_d16, my_stage_u32 + 1024, n0 + 64 * (kp + 1) + j0, row0);
                    bulk_commit();
                }
            }
        }
        buf ^= 1;
        if (buf == 0) tphase ^= 1u;
    }
    if (lane == 0) bulk_wait_read<0>();   // staged rows have left shared memory before the CTA exits (the writes
                                          // themselves are complete when the grid is)
}

template <typename OutT, int EPI, int KIND = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(EPI == EPI_ACT_ROT ? kRotThreads : kThreads, 1)
gemm_i8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_d, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;   // same offset in both CTAs of the pair
    uint8_t* sm = smem_raw + (base - raw_addr);
    const int S = p.stages;
    const int BN = p.bn;
    const int KS = p.ksub;
    const uint32_t a_bytes = BM * BK;                     // one 128-byte K box of this CTA's A rows
    const uint32_t b_bytes = (uint32_t)(BN / 2) * BK;     // ... and of this CTA's half of the W tile
    const uint32_t stage_bytes = KS * (a_bytes + b_bytes);
    uint8_t* staging = sm;                                 // kEpiWarps x 4 KB of output staging
    const uint32_t sA = base + kStagingBytes;              // S x KS x [128 x 128]
    const uint32_t sB = sA + S * KS * a_bytes;             // S x KS x [bn/2 x 128]
    uint8_t* tail = sm + kStagingBytes + S * stage_bytes;
    const uint32_t bar_full = smem_u32(tail);              // kMaxStages barriers (the leader's are used)
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;  // kMaxStages, one set per CTA
    const uint32_t bar_tfull = bar_empty + 8 * kMaxStages; // 2, per CTA
    const uint32_t bar_tempty = bar_tfull + 16;            // 2 (the leader's are used)
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(tail + 8 * (2 * kMaxStages + 4));
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_ptr_s + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int nclusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 2 * (EPI == EPI_ACT_ROT ? kRotEpiWarps : kEpiWarps));
        }
        *abort_s = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_w);
        if (p.tma_store) prefetch_tmap(&tmap_d);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_ptr_s), 512);
        tmem_relinquish_pair();
    }
    if constexpr (EPI == EPI_ACT_LUT || EPI == EPI_ACT_ROT) {
        // the activation table's hot part into shared memory (a gather from the whole table through L1 costs the epilogue
        // one wavefront per distinct line and made it, not the tensor core, the limit)
        if (warp >= 2) {
            uint16_t* dst = reinterpret_cast<uint16_t*>(staging + kVecOffset + kEpiWarps * 1024);
            for (uint32_t i = threadIdx.x - 64; i < 2 * kActLutHalf; i += blockDim.x - 64)
                dst[i] = __ldg(p.act_lut + act_lut_pattern(i));
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = cluster_id; w < p.num_items && ok; w += nclusters) {
                const WorkItem wi = decode_item(p, w);
                int tm, tn;
                tile_coords(wi.tile, p.tiles_m, p.tiles_n, tm, tn, p.group_m ? p.group_m : 8);
                const int row_a = tm * (2 * BM) + (int)rank * BM;
                const int row_w = tn * BN + (int)rank * (BN / 2);
                for (int kb = wi.k0; kb < wi.k0 + wi.kn; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_s, ST_TIMEOUT_EMPTY)) { ok = false; break; }
                    if (leader) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * KS * (a_bytes + b_bytes));
                    const uint32_t full = mapa_shared(bar_full + 8 * stage, 0);
                    for (int ks = 0; ks < KS; ++ks) {
                        tma_load_2d_pair(sA + (stage * KS + ks) * a_bytes, &tmap_a, (kb * KS + ks) * BK, row_a, full);
                        tma_load_2d_pair(sB + (stage * KS + ks) * b_bytes, &tmap_w, (kb * KS + ks) * BK, row_w, full);
                    }
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA) ----------------
        // One thread feeds the tensor cores of both SMs. An MMA of this shape lasts 128 cycles and the tensor core
        // queues only a few; a lone thread retires a dependent instruction every few cycles and a barrier
        // operation costs it on the order of a hundred. The loop is therefore kept to a few dozen instructions per
        // stage: descriptor low words advance by adds, nothing 64-bit, one commit (its arrival multicast to both
        // CTAs), no fence between stages (TMA writes and MMA reads are async-proxy accesses ordered by the
        // mbarrier itself), and stages of two K boxes halve the barrier traffic per MMA.
        if (leader && lane == 0) {
            const uint32_t a_lo0 = umma_desc_lo(sA), b_lo0 = umma_desc_lo(sB);
            const uint32_t a_sub = a_bytes >> 4, b_sub = b_bytes >> 4;        // next K box of a stage
            const uint32_t a_step = KS * a_sub, b_step = KS * b_sub;          // next stage
            const uint32_t idesc = p.idesc;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t a_lo = a_lo0, b_lo = b_lo0, bar_f = bar_full, bar_e = bar_empty;
            int buf = 0;
            uint32_t tphase = 0;
            bool ok = true;
            for (int w = cluster_id; w < p.num_items && ok; w += nclusters) {
                const int kn = decode_item(p, w).kn;
                if (!mbar_wait(bar_tempty + 8 * buf, tphase ^ 1u, abort_s, ST_TIMEOUT_TMEM_EMPTY)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256;
                for (int kb = 0; kb < kn; ++kb) {
                    if (!mbar_try_wait(bar_f, phase)) {
                        if (!mbar_wait(bar_f, phase, abort_s, ST_TIMEOUT_FULL)) { ok = false; break; }
                    }
                    {
                        umma_pair_lo<KIND>(d_tmem, a_lo, b_lo, idesc, kb);
                        umma_pair_lo<KIND>(d_tmem, a_lo + 2, b_lo + 2, idesc, 1);   // +32 bytes inside the swizzle row
                        umma_pair_lo<KIND>(d_tmem, a_lo + 4, b_lo + 4, idesc, 1);
                        umma_pair_lo<KIND>(d_tmem, a_lo + 6, b_lo + 6, idesc, 1);
                        if (KS == 2) {
                            const uint32_t a2 = a_lo + a_sub, b2 = b_lo + b_sub;
                            umma_pair_lo<KIND>(d_tmem, a2, b2, idesc, 1);
                            umma_pair_lo<KIND>(d_tmem, a2 + 2, b2 + 2, idesc, 1);
                            umma_pair_lo<KIND>(d_tmem, a2 + 4, b2 + 4, idesc, 1);
                            umma_pair_lo<KIND>(d_tmem, a2 + 6, b2 + 6, idesc, 1);
                        }
                    }
                    umma_commit_pair(bar_e);   // the stage is free in both CTAs once these MMAs have read it
                    ++stage, a_lo += a_step, b_lo += b_step, bar_f += 8, bar_e += 8;
                    if (stage == S) stage = 0, phase ^= 1u, a_lo = a_lo0, b_lo = b_lo0, bar_f = bar_full, bar_e = bar_empty;
                }
                if (!ok) break;
                umma_commit_pair(bar_tfull + 8 * buf);   // accumulator complete: both epilogues may drain it
                buf ^= 1;
                if (buf == 0) tphase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue (both CTAs, 8 warps) ----------------
        if constexpr (EPI == EPI_ACT_ROT) {
            epilogue_rot(p, &tmap_d, staging, tail, bar_tfull, bar_tempty, tmem_base, abort_s, (int)rank, cluster_id, nclusters, warp,
                         lane);
        } else {
        constexpr int kEsz = EPI == EPI_ACC ? 4 : (int)sizeof(OutT);
        constexpr bool kStageVec = kEsz == 2;            // 2-byte outputs: 2 KB chunk + 1.5 KB of per-column vectors
        const int ew = warp - 2;
        const int quad = warp & 3;               // TMEM lane quarter this warp may read
        const int half = ew >> 2;                // which half of the 32-column chunks
        const int nchunks = BN / 32;
        constexpr int kVecBytes = EPI == EPI_RESID ? 1536 : 1024;       // ws[128] | bias[128] | rscale[128] (residual form only)
        uint8_t* my_stage = staging + ew * (kStageVec ? 2048 : 4096);
        const uint32_t my_stage_u32 = smem_u32(my_stage);
        float* my_vec = reinterpret_cast<float*>(staging + kVecOffset + ew * kVecBytes);
        const uint16_t* lut_sm = reinterpret_cast<const uint16_t*>(staging + kVecOffset + kEpiWarps * 1024);   // EPI_ACT_LUT only
        int buf = 0;
        uint32_t tphase = 0;
        for (int w = cluster_id; w < p.num_items; w += nclusters) {
            const WorkItem wi = decode_item(p, w);
            int tm, tn;
            tile_coords(wi.tile, p.tiles_m, p.tiles_n, tm, tn, p.group_m ? p.group_m : 8);
            const int n0 = tn * BN;
            const int row0 = tm * (2 * BM) + (int)rank * BM + quad * 32;
            const int row = row0 + lane;
            const bool row_ok = row < p.M;
            const int rrow = row_ok ? row : p.M - 1;     // rows past M compute on the last row; their output is clipped
            const float xs_r = EPI == EPI_ACC ? 0.f : p.xs ? p.xs[rrow] : 1.f;
            const bool staged = kStageVec && p.tma_store;
            if (staged) {
                // this warp's columns of ws / bias / rscale, fetched while the mainloop still runs
                __syncwarp();
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int n = n0 + (half + 2 * k) * 32 + lane;
                    const bool in = n < p.N && half + 2 * k < nchunks;
                    my_vec[32 * k + lane] = in ? p.ws[n] : 0.f;
                    my_vec[128 + 32 * k + lane] = (in && p.bias) ? to_f<OutT>(reinterpret_cast<const OutT*>(p.bias)[n]) : 0.f;
                    if (EPI == EPI_RESID)
                        my_vec[256 + 32 * k + lane] = !in ? 0.f : p.rscale ? to_f<OutT>(reinterpret_cast<const OutT*>(p.rscale)[n]) : 1.f;
                }
                __syncwarp();
            }
            if (!mbar_wait_warp_relaxed(bar_tfull + 8 * buf, tphase, abort_s, ST_TIMEOUT_TMEM_FULL)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + buf * 256 + ((uint32_t)(quad * 32) << 16);
            // two register sets: the load of the next chunk is in flight while this one is processed
            uint32_t ra[32], rb[32];
            auto emit = [&](const uint32_t (&r)[32], int c) {
                const int col0 = n0 + c * 32;
                if (col0 >= p.N) return;
                if (p.tma_store) {
                    if constexpr (kStageVec) {
                        uint4 pk[4];
                        chunk_compute16<OutT, EPI, 128, KIND>(p, r, rrow, col0, xs_r, my_vec + 32 * ((c - half) >> 1), pk, lut_sm);
                        if (lane == 0) bulk_wait_read<0>();   // the previous chunk's store has read the buffer
                        __syncwarp();
                        chunk_write16(pk, my_stage, lane);
                    } else {
                        if (lane == 0) bulk_wait_read<0>();
                        __syncwarp();
                        chunk_to_smem<OutT, EPI, KIND>(p, r, rrow, col0, xs_r, my_stage, lane);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmap_d, my_stage_u32, col0, row0);
                        bulk_commit();
                    }
                } else if (row_ok) {
                    chunk_direct<OutT, EPI, KIND>(p, r, row, col0, xs_r);
                }
            };
            constexpr bool kResidStaged = EPI == EPI_RESID && kStageVec;
            if (kResidStaged && wi.kind == ITEM_WHOLE) {
                // Residual form. Fetched one by one in front of their eight columns, the residual's 16-byte pieces put four
                // memory latencies per chunk on the drain of a cluster's last tile (this form was 13 us slower than the
                // plain one on the down-projection). Here a chunk's four pieces are requested together, one chunk ahead
                // of their use; the pieces take the place of the second accumulator register set.
                if constexpr (kResidStaged) {
                    auto pieces = [&](uint4 (&rq)[4], int c) {
                        const uint4* rsd = reinterpret_cast<const uint4*>(reinterpret_cast<const OutT*>(p.resid) + (int64_t)rrow * p.N + n0 + c * 32);
#pragma unroll
                        for (int j = 0; j < 4; ++j) rq[j] = rsd[j];
                    };
                    auto finish = [&](const uint32_t (&r)[32], const uint4 (&rq)[4], int c) {
                        uint4 pk[4];
                        chunk_compute16_resid<OutT, 128, KIND>(p, r, rrow, n0 + c * 32, xs_r, my_vec + 32 * ((c - half) >> 1), pk, rq);
                        if (lane == 0) bulk_wait_read<0>();   // the previous chunk's store has read the buffer
                        __syncwarp();
                        chunk_write16(pk, my_stage, lane);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&tmap_d, my_stage_u32, n0 + c * 32, row0);
                            bulk_commit();
                        }
                    };
                    if (staged && p.vec_ok && n0 + BN <= p.N) {
                        uint4 qa[4], qb[4];
                        int c = half;
                        if (c < nchunks) pieces(qa, c);
#pragma unroll 1
                        for (; c < nchunks; c += 4) {
                            tmem_ld32(taddr + c * 32, ra);
                            if (c + 2 < nchunks) pieces(qb, c + 2);
                            tmem_ld_wait();
                            finish(ra, qa, c);
                            if (c + 2 < nchunks) {
                                tmem_ld32(taddr + (c + 2) * 32, ra);
                                if (c + 4 < nchunks) pieces(qa, c + 4);
                                tmem_ld_wait();
                                finish(ra, qb, c + 2);
                            }
                        }
                    } else {      // direct stores, unaligned vectors, a tile that reaches past N
#pragma unroll 1
                        for (int c = half; c < nchunks; c += 2) {
                            if (n0 + c * 32 >= p.N) break;
                            tmem_ld32(taddr + c * 32, ra);
                            tmem_ld_wait();
                            emit(ra, c);
                        }
                    }
                }
            } else if (!kResidStaged && wi.kind == ITEM_WHOLE) {
                int c = half;
                if (c < nchunks) tmem_ld32(taddr + c * 32, ra);
#pragma unroll 1
                for (; c < nchunks; c += 4) {
                    tmem_ld_wait();
                    if (c + 2 < nchunks) tmem_ld32(taddr + (c + 2) * 32, rb);
                    emit(ra, c);
                    if (c + 2 < nchunks) {
                        tmem_ld_wait();
                        if (c + 4 < nchunks) tmem_ld32(taddr + (c + 4) * 32, ra);
                        emit(rb, c + 2);
                    }
                }
            } else {
                // A slice of a split tile adds its raw accumulators into the tile's int32 buffer in global scratch with
                // atomic adds (integer sums do not depend on the order); the slice that arrives last at a chunk's counter
                // reads the total, leaves buffer and counter at zero for the next launch, and runs the epilogue
                // (release / acquire through the fences around the counter).
#pragma unroll 1
                for (int c = half; c < nchunks; c += 2) {
                    tmem_ld32(taddr + c * 32, ra);
                    tmem_ld_wait();
                    if (n0 + c * 32 >= p.N) continue;
                    const int sub = ((int)rank * 4 + quad) * 8 + c;
                    int* sum = p.partials + ((size_t)wi.slot * kCountersPerSlot + sub) * 1024 + lane;   // [32 values][32 lanes]
#pragma unroll
                    for (int j = 0; j < 32; ++j) atomicAdd(sum + 32 * j, (int)ra[j]);
                    __threadfence();
                    __syncwarp();
                    int* cnt = p.scratch + wi.slot * kCountersPerSlot + sub;
                    int old = 0;
                    if (lane == 0) old = atomicAdd(cnt, 1);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old != p.splits - 1) continue;
                    if (lane == 0) *cnt = 0;
                    __threadfence();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        ra[j] = (uint32_t)__ldcg(sum + 32 * j);
                        __stcg(sum + 32 * j, 0);
                    }
                    emit(ra, c);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * buf, 0));
            buf ^= 1;
            if (buf == 0) tphase ^= 1u;
        }
        if (p.tma_store && lane == 0) bulk_wait_read<0>();   // staged rows have left shared memory before the CTA exits
                                                             // (the writes themselves are complete when the grid is)
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // nobody leaves while the peer may still signal its barriers or read its tiles
    if (*abort_s != 0) {
        // a wait ran out: leave time for copies and MMAs still in flight, then report
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicCAS(&g_kernel_status, 0, *abort_s);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---- small problems: one CTA per 128 x bn tile --------------------------------------------------------------------------
// A launch of the persistent CTA-pair kernel costs about 12 us before its size matters (cluster launch with the full shared
// memory, two cluster barriers, 512 tensor-memory columns, a ring of 64 KB stages): for problems of a few hundred Mop (the
// cross-attention K/V projections of the SDXL U-Net: 154 rows) that is the whole time. This kernel is the same dataflow
// without the pair: one CTA per tile, tcgen05.mma.cta_group::1 (M = 128, N = bn <= 128, K = 32), a ring of 128-byte K boxes
// of A (128 rows) and W (bn rows), one accumulator of bn tensor-memory columns, four epilogue warps (one per lane quarter)
// that store straight to D with the arithmetic of the large kernel. Warp 0 loads, warp 1 issues the MMAs.
constexpr int kSmallThreads = 192;
constexpr int kSmallMaxStages = 8;
template <typename OutT, int EPI>
__global__ void __launch_bounds__(kSmallThreads, 1)
gemm_i8_small_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw_addr);
    const int S = p.stages, BN = p.bn;
    const uint32_t a_bytes = BM * BK, b_bytes = (uint32_t)BN * BK;
    const uint32_t sA = base, sB = sA + S * a_bytes;
    uint8_t* tail = sm + S * (a_bytes + b_bytes);
    const uint32_t bar_full = smem_u32(tail), bar_empty = bar_full + 8 * kSmallMaxStages, bar_tfull = bar_empty + 8 * kSmallMaxStages;
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(tail + 8 * (2 * kSmallMaxStages + 1));
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_ptr_s + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tmem_cols = BN <= 32 ? 32u : BN <= 64 ? 64u : 128u;
    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        mbar_init(bar_tfull, 1);
        *abort_s = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_ptr_s), tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;
    const int tm = blockIdx.x % p.tiles_m, tn = blockIdx.x / p.tiles_m;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < p.k_iters; ++kb) {
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_s, ST_TIMEOUT_EMPTY)) break;
                mbar_arrive_expect_tx(bar_full + 8 * stage, a_bytes + b_bytes);
                tma_load_2d(sA + stage * a_bytes, &tmap_a, kb * BK, tm * BM, bar_full + 8 * stage);
                tma_load_2d(sB + stage * b_bytes, &tmap_w, kb * BK, tn * BN, bar_full + 8 * stage);
                if (++stage == S) stage = 0, phase ^= 1u;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = p.idesc;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < p.k_iters; ++kb) {
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_s, ST_TIMEOUT_FULL)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da = umma_desc_sw128(sA + stage * a_bytes), db = umma_desc_sw128(sB + stage * b_bytes);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) umma_i8(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);   // +32 bytes per step
                umma_commit(bar_empty + 8 * stage);
                if (++stage == S) stage = 0, phase ^= 1u;
            }
            if (ok) umma_commit(bar_tfull);
        }
    } else {
        const int quad = warp & 3;               // TMEM lane quarter this warp may read (warps 2..5 cover all four)
        const int row = tm * BM + quad * 32 + lane;
        const bool row_ok = row < p.M;
        const float xs_r = EPI == EPI_ACC ? 0.f : (p.xs && row_ok) ? p.xs[row] : 1.f;
        if (mbar_wait_warp_relaxed(bar_tfull, 0, abort_s, ST_TIMEOUT_TMEM_FULL)) {
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
            uint32_t r[32];
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col0 = tn * BN + c * 32;
                if (col0 >= p.N) break;
                tmem_ld32(taddr + c * 32, r);
                tmem_ld_wait();
                if (row_ok) chunk_direct<OutT, EPI, 0>(p, r, row, col0, xs_r);
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_s != 0) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);      // leave time for copies and MMAs still in flight, then report
        if (threadIdx.x == 0) atomicCAS(&g_kernel_status, 0, *abort_s);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// ---- host side ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::atomic<EncodeTiledFn> fn{nullptr};
    EncodeTiledFn f = fn.load(std::memory_order_acquire);
    if (f) return f;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !sym)
        return nullptr;
    f = reinterpret_cast<EncodeTiledFn>(sym);
    fn.store(f, std::memory_order_release);
    return f;
}

bool encode_operand_tmap(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols, int box_rows);
bool encode_output_tmap(CUtensorMap* tm, void* ptr, int64_t M, int64_t N, int esz);

// Encoded tensor maps depend only on address, shape and box, not on the data: an inference loop presents the same
// buffers again and again, so each thread remembers its last few (a map is 128 bytes; the driver call that encodes
// one takes about a microsecond of host time, three per GEMM call).
struct TmapKey {
    const void* ptr;
    int64_t d0, d1, pitch;
    int box0, box1, kind;     // kind: element type and swizzle
    bool operator==(const TmapKey& o) const {
        return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && pitch == o.pitch && box0 == o.box0 && box1 == o.box1 && kind == o.kind;
    }
};
struct TmapCache {
    static constexpr int kSlots = 16;
    TmapKey key[kSlots] = {};
    CUtensorMap map[kSlots];
    bool used[kSlots] = {};
    int next = 0;
    const CUtensorMap* find(const TmapKey& k) const {
        for (int i = 0; i < kSlots; ++i)
            if (used[i] && key[i] == k) return &map[i];
        return nullptr;
    }
    void put(const TmapKey& k, const CUtensorMap& m) {
        key[next] = k, map[next] = m, used[next] = true;
        next = (next + 1) % kSlots;
    }
};
thread_local TmapCache g_tmaps;

// Tensor map of a row-major int8 matrix [rows, cols] (cols contiguous), box 128 bytes x box_rows, 128-byte swizzle.
// Rows and columns beyond the matrix read as zero.
bool make_operand_tmap(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
    const TmapKey k{ptr, cols, rows, cols, BK, box_rows, 0};
    if (const CUtensorMap* hit = g_tmaps.find(k)) { *tm = *hit; return true; }
    if (!encode_operand_tmap(tm, ptr, rows, cols, box_rows)) return false;
    g_tmaps.put(k, *tm);
    return true;
}
bool encode_operand_tmap(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Tensor map of the output [M, N] for stores of 32 x 32-element boxes: 64-byte rows (64-byte swizzle) for 2-byte
// elements, 128-byte rows (128-byte swizzle) for 4-byte elements.
bool make_output_tmap(CUtensorMap* tm, void* ptr, int64_t M, int64_t N, int esz) {
    const TmapKey k{ptr, N, M, N * esz, 32, 32, esz == 2 ? 1 : 2};
    if (const CUtensorMap* hit = g_tmaps.find(k)) { *tm = *hit; return true; }
    if (!encode_output_tmap(tm, ptr, M, N, esz)) return false;
    g_tmaps.put(k, *tm);
    return true;
}
// The rotating epilogue's map: bf16 output, boxes of 16 columns x 32 rows (32-byte rows, 32-byte swizzle)
bool make_output_tmap16(CUtensorMap* tm, void* ptr, int64_t M, int64_t N) {
    const TmapKey k{ptr, N, M, N * 2, 16, 32, 3};
    if (const CUtensorMap* hit = g_tmaps.find(k)) { *tm = *hit; return true; }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)(N * 2)};
    const cuuint32_t box[2] = {16, 32};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    g_tmaps.put(k, *tm);
    return true;
}
bool encode_output_tmap(CUtensorMap* tm, void* ptr, int64_t M, int64_t N, int esz) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)(N * esz)};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t estr[2] = {1, 1};
    return enc(tm, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, ptr, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, esz == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Upper bound on the CTA pairs a GEMM launch occupies (0 = every SM pair of the device); see gpu_int8_gemm_set_cluster_limit.
std::atomic<int> g_cluster_limit{0};

int device_sm_count(int dev) {
    static int count[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    int& c = count[dev & 63];
    if (c == 0) cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev);
    return c;
}

template <typename OutT, int EPI, int KIND = 0>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& td, const GemmParams& p, int grid,
                cudaStream_t st) {
    auto kern = gemm_i8_pair_kernel<OutT, EPI, KIND>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured.fetch_or(bit, std::memory_order_release);
    }
    kern<<<grid, EPI == EPI_ACT_ROT ? kRotThreads : kThreads, kSmemBytes, st>>>(ta, tw, td, p);
    KCHECK();
    return 0;
}
template <typename OutT>
int launch_pair_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& td, const GemmParams& p,
                    int grid, cudaStream_t st) {
    switch (epi) {
        case EPI_PLAIN: return launch_pair<OutT, EPI_PLAIN>(ta, tw, td, p, grid, st);
        case EPI_RESID: return launch_pair<OutT, EPI_RESID>(ta, tw, td, p, grid, st);
        case EPI_ACT: return launch_pair<OutT, EPI_ACT>(ta, tw, td, p, grid, st);
        case EPI_ACT_LUT:
            if constexpr (std::is_same<OutT, bf16>::value) return launch_pair<bf16, EPI_ACT_LUT>(ta, tw, td, p, grid, st);
            return -200;
        case EPI_ACT_ROT:
            if constexpr (std::is_same<OutT, bf16>::value) return launch_pair<bf16, EPI_ACT_ROT>(ta, tw, td, p, grid, st);
            return -200;
        default: return -200;
    }
}

template <typename OutT, int EPI>
int launch_small(const CUtensorMap& ta, const CUtensorMap& tw, const GemmParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = gemm_i8_small_kernel<OutT, EPI>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured.fetch_or(bit, std::memory_order_release);
    }
    kern<<<grid, kSmallThreads, smem, st>>>(ta, tw, p);
    KCHECK();
    return 0;
}
template <typename OutT>
int launch_small_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tw, const GemmParams& p, int grid, size_t smem,
                     cudaStream_t st) {
    switch (epi) {
        case EPI_PLAIN: return launch_small<OutT, EPI_PLAIN>(ta, tw, p, grid, smem, st);
        case EPI_RESID: return launch_small<OutT, EPI_RESID>(ta, tw, p, grid, smem, st);
        case EPI_ACT: return launch_small<OutT, EPI_ACT>(ta, tw, p, grid, smem, st);
        default: return -200;
    }
}

// Scratch of the K-split forms (split few-tile problems, streamed tail): per device and stream, one buffer allocated on
// first need and kept (a stream-ordered allocation per call cost more host time than the split saves). Counters and sums
// are zero between launches: the buffer is cleared on the caller's stream before its first use, every kernel leaves it at
// zero, and after a kernel has reported a bounded wait that ran out (gpu_kernels_status) it is cleared again before
// the next use. A stream beyond the few slots, a failed allocation or a stream under capture that has no buffer yet
// simply runs without the split.
constexpr int kWorkspaceSlots = 40;                       // tiles of 256 x 256 int32 sums (at most half the clusters' worth)
constexpr size_t kWorkspaceCounterBytes = 1 << 16;        // counters first, sums behind them
constexpr size_t kSplitWorkspaceBytes = (size_t)kWorkspaceSlots * 256 * 256 * 4 + kWorkspaceCounterBytes;
std::atomic<uint64_t> g_workspace_epoch{1};               // raised when a kernel may have left scratch behind
int* split_workspace(int dev, cudaStream_t st, size_t need) {
    struct Slot { cudaStream_t st; int* buf; bool used; uint64_t clean_epoch; };
    static Slot slots[64][4];
    static std::mutex mu;
    if (need > kSplitWorkspaceBytes) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    Slot* s = slots[dev & 63];
    Slot* hit = nullptr;
    for (int i = 0; i < 4 && !hit; ++i)
        if (s[i].used && s[i].st == st) hit = &s[i];
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    const uint64_t epoch = g_workspace_epoch.load(std::memory_order_acquire);
    if (!hit || hit->clean_epoch != epoch) {
        if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
            (void)cudaGetLastError();
            return nullptr;   // neither an allocation nor a clear while the stream is being captured
        }
    }
    for (int i = 0; i < 4 && !hit; ++i) {
        if (s[i].used) continue;
        void* b = nullptr;
        if (cudaMalloc(&b, kSplitWorkspaceBytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        s[i] = {st, reinterpret_cast<int*>(b), true, 0};
        hit = &s[i];
    }
    if (!hit) return nullptr;
    if (hit->clean_epoch != epoch) {
        if (cudaMemsetAsync(hit->buf, 0, kSplitWorkspaceBytes, st) != cudaSuccess) {   // ordered before the kernel that uses it
            (void)cudaGetLastError();
            return nullptr;
        }
        hit->clean_epoch = epoch;
    }
    return hit->buf;
}

// Column-tile width: the candidate whose rounds x (width + fixed per-tile cost) is smallest, so that a shape leaving
// the last round nearly empty at 256 takes a narrower tile instead; narrower tiles read A from L2 once more per column
// tile, and on large shapes the L2 -> SM path, not the tensor core, is what the kernel waits for (up-projection: 113 us
// at 256 against 118 at 224 and 124 at 192, although 224 has the smaller product), hence the mild penalty on width lost.
// (Launching only as many CTA pairs as the round count needs, 68 instead of 74 for 816 tiles in 12 rounds, leaves SMs idle
// and raises the power-capped clock by about 1 %, but the step was 0.7 % slower: not done.)
int choose_bn(int64_t M, int64_t N, int clusters) {
    const int64_t tm = (M + 2 * BM - 1) / (2 * BM);
    int best = 256;
    double best_cost = 1e30;
    for (int bn = 256; bn >= 64; bn -= 32) {
        const int64_t tiles = tm * ((N + bn - 1) / bn);
        const int64_t rounds = (tiles + clusters - 1) / clusters;
        const double cost = (double)rounds * (bn + 32) * (1.0 + 0.4 * (256 - bn) / 256.0);
        if (cost < best_cost) best_cost = cost, best = bn;
    }
    return best;
}

int run_gemm(int epi, const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias,
             const void* rscale, const void* resid, void* D, int64_t M, int64_t N, int64_t K, int out_dt, int act,
             cudaStream_t st, float* amax_part = nullptr) {
    if (M == 0 || N == 0) return 0;
    if (K == 0) return epi == EPI_RESID ? -201 : 0;  // the reference declines K == 0 for the residual form only
    if (epi == EPI_RESID && (!rscale || !resid)) return -201;
    if (epi != EPI_ACC && (out_dt < 0 || out_dt > 2)) return epi == EPI_RESID ? -201 : -200;
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return -200;
    // like the reference, rows must at least be a whole number of 8-byte pieces (its narrowest tile configurations,
    // csrc/vendor/cutlass_gemm_int8.cu:265-267); it answers anything else with its "no configuration" code
    if ((K % 8) != 0) return epi == EPI_RESID ? -201 : -200;
    int dev = 0;
    cudaGetDevice(&dev);
    const bool rot = epi == EPI_ACT_ROT;
    // the rotating epilogue exists on the tensor-core kernel only: bf16 rows of whole 256-column rotation groups
    if (rot && (out_dt != DT_BF16 || (N % 256) != 0 || (K % 16) != 0 || (((uintptr_t)A | (uintptr_t)W | (uintptr_t)D) & 15) ||
                !amax_part || act < 1 || act > 3))
        return -208;
    // TMA needs 16-byte aligned bases and row pitch; what it cannot address takes the CUDA-core kernel
    if ((K % 16) != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) {
        SkinnyParams sp{A, W, xs, ws, bias, rscale, resid, D, (int)M, (int)N, (int)K, act};
        return launch_generic_gemm(epi, sp, out_dt, st);
    }
    if (!rot && skinny_gemm_applies(M, N, K)) {
        SkinnyParams sp{A, W, xs, ws, bias, rscale, resid, D, (int)M, (int)N, (int)K, act};
        return launch_skinny_gemm(epi, sp, out_dt, device_sm_count(dev), st);
    }
    int clusters = device_sm_count(dev) / 2;
    if (const int lim = g_cluster_limit.load(std::memory_order_relaxed); lim > 0 && lim < clusters) clusters = lim;
    GemmParams p{};
    p.xs = xs, p.ws = ws, p.bias = bias, p.rscale = rscale, p.resid = resid, p.D = D;
    p.M = (int)M, p.N = (int)N, p.K = (int)K;
    p.act = act;
    p.act_lut = nullptr;
    p.amax_part = amax_part;
    // Small problems (the pair kernel's launch alone would be most of their time): one CTA per 128 x bn tile, the tile
    // width chosen so that about a hundred CTAs or more share the work.
    // (a few tiles with a long K stay with the pair kernel, which cuts them along K over all SMs)
    int small_bn = 128;
    const int small_tm = (int)((M + BM - 1) / BM);
    while (small_bn > 32 && (int64_t)small_tm * ((N + small_bn - 1) / small_bn) < 96) small_bn >>= 1;
    const int64_t small_tiles = (int64_t)small_tm * ((N + small_bn - 1) / small_bn);
    const double ops = 2.0 * (double)M * (double)N * (double)K;
    // measured on the SDXL shapes: below 2 Gop always (154 x 2048 x 640: 10.2 against 13.5 us in kernel); up to 8 Gop when
    // the tiles fit the SMs in little more than one wave (2048 x 1280 x 1280, 160 tiles: 14.9 against 16.5 us; 8192 x 640 x
    // 640, 320 tiles: 21.7 against 18.8, so not there)
    const bool small = !rot && ((ops < kSmallProblemOps && (K <= 4096 || small_tiles >= 64)) ||
                                (ops < 4.0 * kSmallProblemOps && K <= 4096 && small_tiles * 5 <= (int64_t)device_sm_count(dev) * 6));
    if (small) {
        const int tiles_m = small_tm;
        const int bn = small_bn;
        auto al16s = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
        p.vec_ok = (N % 8 == 0) && al16s(D) && al16s(ws) && al16s(bias) && al16s(rscale) && al16s(resid);
        p.tma_store = 0;
        p.bn = bn, p.ksub = 1;
        p.k_iters = (int)((K + BK - 1) / BK);
        p.tiles_m = tiles_m, p.tiles_n = (int)((N + bn - 1) / bn), p.num_tiles = p.tiles_m * p.tiles_n;
        // ring depth: the whole K if it fits; half the SM's shared memory when there are more tiles than SMs, so that two
        // CTAs share an SM
        const int stage_bytes = BM * BK + bn * BK;
        const int budget = (p.num_tiles > device_sm_count(dev) ? kSmemBytes / 2 : kSmemBytes) - 1024 - 256;
        p.stages = budget / stage_bytes;
        if (p.stages > kSmallMaxStages) p.stages = kSmallMaxStages;
        if (p.stages > p.k_iters) p.stages = p.k_iters;
        p.idesc = umma_idesc_i8(BM, bn);
        CUtensorMap ta, tw;
        if (!make_operand_tmap(&ta, A, M, K, BM) || !make_operand_tmap(&tw, W, N, K, bn)) return -203;
        const size_t smem = 1024 + (size_t)p.stages * (BM * BK + bn * BK) + 256;
        if (epi == EPI_ACC) return launch_small<float, EPI_ACC>(ta, tw, p, p.num_tiles, smem, st);
        if (out_dt == DT_F32) return launch_small_epi<float>(epi, ta, tw, p, p.num_tiles, smem, st);
        if (out_dt == DT_F16) return launch_small_epi<half>(epi, ta, tw, p, p.num_tiles, smem, st);
        return launch_small_epi<bf16>(epi, ta, tw, p, p.num_tiles, smem, st);
    }
    const int esz = epi == EPI_ACC ? 4 : (out_dt == DT_F32 ? 4 : 2);
    auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    p.vec_ok = (N % 8 == 0) && al16(D) && al16(ws) && al16(bias) && al16(rscale) && al16(resid);
    p.tma_store = al16(D) && ((N * esz) % 16 == 0);
    // large bf16 outputs take the activation from the table (the staged-output path keeps its hot part in shared memory)
    if (epi == EPI_ACT && out_dt == DT_BF16 && M * N >= (1 << 20) && p.tma_store) {
        if (int rc = act_lut_ptr(act, st, &p.act_lut)) return rc;
        epi = EPI_ACT_LUT;
    }
    if (rot)
        if (int rc = act_lut_ptr(act, st, &p.act_lut)) return rc;
    p.ksub = K <= BK ? 1 : 2;
    p.k_iters = (int)((K + p.ksub * BK - 1) / (p.ksub * BK));
    const int bn = rot ? 256 : choose_bn(M, N, clusters);
    p.bn = bn;
    p.idesc = umma_idesc_i8(2 * BM, bn);
    const int stage_bytes = p.ksub * (BM * BK + (bn / 2) * BK);
    const int stages = (kSmemBytes - 1024 - kTailBytes - kStagingBytes) / stage_bytes;
    p.stages = stages > kMaxStages ? kMaxStages : stages;
    p.tiles_m = (int)((M + 2 * BM - 1) / (2 * BM));
    p.tiles_n = (int)((N + bn - 1) / bn);
    p.num_tiles = p.tiles_m * p.tiles_n;
    {   // Bands whose rows of A (M x K bytes) stay in L2 while W and D stream past, as few of them as that allows: W is
        // then read from DRAM once per band. A small W stays in L2 by itself, and bands of eight rows (about a square of
        // tiles per wave) serve both operands best (16896 x 3072 x 3072: 110 against 113 us with tall bands).
        const int64_t bands = (M * K + kResidentOperandBytes - 1) / kResidentOperandBytes;
        const int gm = (int)((p.tiles_m + bands - 1) / bands);
        p.group_m = (N * K > kResidentOperandBytes / 2 && gm > 12) ? gm : 8;      // a little taller than eight makes no difference
    }
    CUtensorMap ta, tw, td;
    if (!make_operand_tmap(&ta, A, M, K, BM) || !make_operand_tmap(&tw, W, N, K, bn / 2)) return -203;
    if (rot) {
        if (!make_output_tmap16(&td, D, M, N)) return -203;
    } else if (p.tma_store) {
        if (!make_output_tmap(&td, D, M, N, esz)) return -203;
    } else {
        td = ta;  // unused
    }
    // K split: a problem with fewer tiles than clusters and a long K (few rows, few columns) is cut along K so that
    // more SMs stream it; partial sums meet by atomic adds and the slice that arrives last runs the epilogue. Measured
    // on B200: worth it only when every slice keeps at least eight stages. Cutting the ragged last round of a many-round
    // problem instead (stream-K: the last rounds' tiles dealt out in K stages, tiles shared by two clusters meeting
    // through scratch) was built and measured slower than whole tiles on both benchmark linears (121 against 116 us on the
    // up-projection; 155 against 121 us on the down-projection, where clusters no longer walk K in step and the L2 has to
    // hold both matrices), so many-round problems run whole tiles only.
    p.whole_tiles = p.num_tiles, p.splits = 0, p.kps = p.k_iters, p.num_items = p.num_tiles;
    p.scratch = nullptr, p.partials = nullptr;
    const int rem = p.num_tiles % clusters;
    if (!rot && rem > 0 && p.num_tiles < clusters && 2 * rem <= clusters && p.k_iters >= 16) {
        int splits = clusters / rem;
        if (splits > p.k_iters / 8) splits = p.k_iters / 8;
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
        const int kps = (p.k_iters + splits - 1) / splits;
        splits = (p.k_iters + kps - 1) / kps;
        int* wsp = splits >= 2 && rem <= kWorkspaceSlots ? split_workspace(dev, st, kSplitWorkspaceBytes) : nullptr;
        if (wsp) {
            p.scratch = wsp;
            p.partials = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(wsp) + kWorkspaceCounterBytes);
            p.whole_tiles = p.num_tiles - rem, p.splits = splits, p.kps = kps;
            p.num_items = p.whole_tiles + rem * splits;
        }
    }
    const int grid = 2 * (p.num_items < clusters ? p.num_items : clusters);
    int rc;
    if (epi == EPI_ACC) rc = launch_pair<float, EPI_ACC>(ta, tw, td, p, grid, st);
    else if (out_dt == DT_F32) rc = launch_pair_epi<float>(epi, ta, tw, td, p, grid, st);
    else if (out_dt == DT_F16) rc = launch_pair_epi<half>(epi, ta, tw, td, p, grid, st);
    else rc = launch_pair_epi<bf16>(epi, ta, tw, td, p, grid, st);
    return rc;
}

// ---- weight-only int8 linear (the text encoders' path) ---------------------------------------------------------------
// int8 codes are exact in bf16, so W goes to the tensor cores as bf16 without loss; the f32 activation goes as two bf16
// terms (hi + lo = 16 significant bits), one GEMM pass each into f32 accumulators: close to an fp32 product at tensor-core
// speed. The kernel is the int8 one with kind::f16 MMAs (bf16 operands are addressed as rows of 2 K bytes).
__global__ void __launch_bounds__(256) widen_i8_bf16_kernel(const int8_t* __restrict__ q, bf16* __restrict__ out, int64_t n16) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n16) return;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(q) + i);
    const int8_t* b = reinterpret_cast<const int8_t*>(&v);
    __nv_bfloat162 o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = __floats2bfloat162_rn((float)b[2 * e], (float)b[2 * e + 1]);
    reinterpret_cast<uint4*>(out)[2 * i] = *reinterpret_cast<const uint4*>(&o[0]);
    reinterpret_cast<uint4*>(out)[2 * i + 1] = *reinterpret_cast<const uint4*>(&o[4]);
}

// D[M,N] (f32) = [resid +] (A[M,K] . W[N,K]^T) * ws[n], A and W bf16 row-major, K % 8 == 0, 16-byte aligned.
int run_gemm_bf16(bool add, const void* A, const void* W, const float* ws, float* D, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    if (M == 0 || N == 0 || K == 0) return 0;
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX / 2) return -200;
    if ((K % 8) != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)D & 15)) return -202;
    int dev = 0;
    cudaGetDevice(&dev);
    int clusters = device_sm_count(dev) / 2;
    if (const int lim = g_cluster_limit.load(std::memory_order_relaxed); lim > 0 && lim < clusters) clusters = lim;
    const int64_t Kb = 2 * K;                                   // bytes per row
    GemmParams p{};
    p.xs = nullptr, p.ws = ws, p.bias = nullptr, p.rscale = nullptr, p.resid = add ? D : nullptr, p.D = D;
    p.M = (int)M, p.N = (int)N, p.K = (int)Kb;
    auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    p.vec_ok = (N % 8 == 0) && al16(ws);
    p.tma_store = (N * 4) % 16 == 0;
    p.ksub = Kb <= BK ? 1 : 2;
    p.k_iters = (int)((Kb + p.ksub * BK - 1) / (p.ksub * BK));
    const int bn = choose_bn(M, N, clusters);
    p.bn = bn;
    p.idesc = umma_idesc_bf16(2 * BM, bn);
    const int stage_bytes = p.ksub * (BM * BK + (bn / 2) * BK);
    const int stages = (kSmemBytes - 1024 - kTailBytes - kStagingBytes) / stage_bytes;
    p.stages = stages > kMaxStages ? kMaxStages : stages;
    p.tiles_m = (int)((M + 2 * BM - 1) / (2 * BM));
    p.tiles_n = (int)((N + bn - 1) / bn);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.whole_tiles = p.num_tiles, p.splits = 0, p.kps = p.k_iters, p.num_items = p.num_tiles;
    CUtensorMap ta, tw, td;
    if (!make_operand_tmap(&ta, A, M, Kb, BM) || !make_operand_tmap(&tw, W, N, Kb, bn / 2)) return -203;
    if (p.tma_store) {
        if (!make_output_tmap(&td, D, M, N, 4)) return -203;
    } else {
        td = ta;
    }
    const int grid = 2 * (p.num_items < clusters ? p.num_items : clusters);
    return add ? launch_pair<float, EPI_RESID, 1>(ta, tw, td, p, grid, st) : launch_pair<float, EPI_PLAIN, 1>(ta, tw, td, p, grid, st);
}

#include "gemm_w6.inl"

}  // namespace

// New: the W6A8 linear without the decoded copy. The reference expands the packed weight to int8 in a scratch buffer
// (gpu_w6_decode, csrc/h3.cu:11-46) and then calls gpu_int8_gemm on it (src/h3.rs:1208-1216); these read the packed rows
// [N, 3K/4] and the e4m3 group scales [N, K/32] directly and expand them in shared memory. Same results as that pair of
// calls, bit for bit. ws = the per-channel scale (s_channel). K must be a multiple of 128, G must be 32 (-206 otherwise).
GPU_API int gpu_w6a8_gemm(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, const float* xs, const float* ws,
                          const void* bias, void* D, int64_t M, int64_t N, int64_t K, int G, int out_dt, void* stream) {
    return run_w6_gemm(EPI_PLAIN, A, Wq6, s_rel, xs, ws, bias, nullptr, nullptr, D, M, N, K, G, out_dt, (cudaStream_t)stream);
}
GPU_API int gpu_w6a8_gemm_residual(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, const float* xs,
                                   const float* ws, const void* bias, const void* rscale, const void* resid, void* D,
                                   int64_t M, int64_t N, int64_t K, int G, int out_dt, void* stream) {
    return run_w6_gemm(EPI_RESID, A, Wq6, s_rel, xs, ws, bias, rscale, resid, D, M, N, K, G, out_dt, (cudaStream_t)stream);
}
// The same with the activation the next quantizer's prologue would apply (the FFN-up linear of the W6A8 video DiT):
// D = out(act(out(acc * xs * ws + bias))), act as in gpu_int8_gemm_act.
GPU_API int gpu_w6a8_gemm_act(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, const float* xs, const float* ws,
                              const void* bias, void* D, int64_t M, int64_t N, int64_t K, int G, int out_dt, int act,
                              void* stream) {
    if (act == ACT_NONE) return gpu_w6a8_gemm(A, Wq6, s_rel, xs, ws, bias, D, M, N, K, G, out_dt, stream);
    if (act < 0 || act > 3) return -204;
    return run_w6_gemm(EPI_ACT, A, Wq6, s_rel, xs, ws, bias, nullptr, nullptr, D, M, N, K, G, out_dt, (cudaStream_t)stream, act);
}
// For tests: the raw int32 accumulators of the fused-unpack GEMM.
GPU_API int gpu_w6a8_gemm_acc_i32(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, int32_t* D, int64_t M,
                                  int64_t N, int64_t K, int G, void* stream) {
    return run_w6_gemm(EPI_ACC, A, Wq6, s_rel, nullptr, nullptr, nullptr, nullptr, nullptr, D, M, N, K, G, 0, (cudaStream_t)stream);
}

// New: the weight-only int8 linear of the text encoders in one call. The reference rotates the f32 activation rows
// (gpu_rotate_rows_f32, csrc/kernels.cu:316-327), dequantizes the whole int8 weight to f32 (gpu_dequant_i8, :330-343) and runs
// an fp32 GEMM with beta 0 or 1 (src/te.rs:493-511). Here: out[M,N] = beta * out + R256(prologue(x)) . (Wq * ws[n])^T with the
// product on the bf16 tensor cores: Wq widens to bf16 exactly, the rotated rows go as hi + lo bf16 terms (two passes, f32
// accumulation), so the result is within about 2^-16 relative of the fp32 product's terms.
//   prologue   PRO_PLAIN, PRO_RMS (norm_w, eps) or PRO_SWIGLU (up_offset) as gpu_rotate_rows_f32 takes them
//   a_scratch  >= 4 * M * K bytes (the reference's rotated-rows buffer has that size), w_scratch >= 2 * N * K bytes
//              (half of the reference's dequantized-weight buffer); both 16-byte aligned
//   beta       0 or 1 (-207 otherwise); K % 256 == 0 (-1); N * 4 bytes a multiple of 16 for the fast store path
GPU_API int gpu_wo8_linear(int prologue, const float* x, int64_t x_stride, int64_t up_offset, const float* norm_w, float eps,
                           const int8_t* Wq, const float* ws, float* out, float beta, void* a_scratch, void* w_scratch, int M,
                           int N, int K, void* stream) {
    if ((K % 256) != 0) return -1;
    if (beta != 0.f && beta != 1.f) return -207;
    if (M <= 0 || N <= 0) return 0;
    if ((((uintptr_t)a_scratch | (uintptr_t)w_scratch | (uintptr_t)Wq) & 15) || !a_scratch || !w_scratch) return -202;
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t* hi = reinterpret_cast<uint8_t*>(a_scratch);
    uint8_t* lo = hi + (size_t)M * K * 2;
    if (int rc = rotate_rows_split(prologue, x, x_stride, up_offset, norm_w, eps, hi, lo, M, K, st)) return rc;
    const int64_t n16 = (int64_t)N * K / 16;
    widen_i8_bf16_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, st>>>(Wq, reinterpret_cast<bf16*>(w_scratch), n16);
    KCHECK();
    if (int rc = run_gemm_bf16(beta == 1.f, hi, w_scratch, ws, out, M, N, K, st)) return rc;
    return run_gemm_bf16(true, lo, w_scratch, ws, out, M, N, K, st);
}

// D[M,N] = (A[M,K] . W[N,K]^T) * xs[m] * ws[n] + bias[n]; replaces the reference's csrc/gemm.cu:123-129.
GPU_API int gpu_int8_gemm(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias, void* D,
                          int64_t M, int64_t N, int64_t K, int out_dt, void* stream) {
    return run_gemm(EPI_PLAIN, A, W, xs, ws, bias, nullptr, nullptr, D, M, N, K, out_dt, 0, (cudaStream_t)stream);
}

// D = resid + rscale[n] * (acc * xs[m] * ws[n] + bias[n]); D may alias resid; csrc/gemm.cu:131-140.
GPU_API int gpu_int8_gemm_residual(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias,
                                   const void* rscale, const void* resid, void* D, int64_t M, int64_t N, int64_t K,
                                   int out_dt, void* stream) {
    return run_gemm(EPI_RESID, A, W, xs, ws, bias, rscale, resid, D, M, N, K, out_dt, 0, (cudaStream_t)stream);
}

// New: the activation the reference applies in the next quantizer's prologue (csrc/kernels.cu:121-130), applied
// here to the rounded linear output: D = out(act(out(acc*xs*ws + bias))). act: 1 gelu-tanh, 2 silu, 3 gelu-erf.
GPU_API int gpu_int8_gemm_act(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias,
                              void* D, int64_t M, int64_t N, int64_t K, int out_dt, int act, void* stream) {
    if (act == ACT_NONE) return gpu_int8_gemm(A, W, xs, ws, bias, D, M, N, K, out_dt, stream);
    if (act < 0 || act > 3) return -204;
    return run_gemm(EPI_ACT, A, W, xs, ws, bias, nullptr, nullptr, D, M, N, K, out_dt, act, (cudaStream_t)stream);
}

// New: gpu_int8_gemm_act whose epilogue also rotates. The reference runs the MLP's second half as GEMM -> quantizer with the
// GELU prologue and the R256 rotation -> GEMM (src/qwen21.rs:378-417; csrc/kernels.cu:121-130,184-258), and the quantizer's
// rotation is what that kernel spends its time on. Here the up-projection's epilogue, which holds one whole rotation group
// of each row (256 columns) in tensor memory, applies the activation and the rotation while the tensor cores run the next
// tile, and leaves   D[m, :] = bf16(R256(act(bf16(acc * xs * ws + bias))))   (bf16 only) together with
// amax_part[N / 64, M]: partial maxima of the unrounded rotated values, four per tile (sign bit: a NaN was among them).
// gpu_quant_rows_rotated turns the two into the codes and scales gpu_quant_rows(prologue = the activation, rotate = 1)
// gives on the plain GEMM's output, bit for bit. N % 256 == 0, K % 16 == 0, 16-byte aligned operands, act 1..3 (-208 otherwise).
GPU_API int gpu_int8_gemm_act_rot(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias, void* D,
                                  float* amax_part, int64_t M, int64_t N, int64_t K, int act, void* stream) {
    return run_gemm(EPI_ACT_ROT, A, W, xs, ws, bias, nullptr, nullptr, D, M, N, K, DT_BF16, act, (cudaStream_t)stream, amax_part);
}

// New, for tests: the raw int32 accumulators D[m,n] = sum_k A[m,k]*W[n,k], which the fused forms never expose.
GPU_API int gpu_int8_gemm_acc_i32(const int8_t* A, const int8_t* W, int32_t* D, int64_t M, int64_t N, int64_t K,
                                  void* stream) {
    return run_gemm(EPI_ACC, A, W, nullptr, nullptr, nullptr, nullptr, nullptr, D, M, N, K, 0, 0, (cudaStream_t)stream);
}

namespace {

// ---- the entry point that allocates nothing ----------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc once they are running: the reference's engine, for one, fills the
// card up to a watermark with its own allocator and then lives inside that budget (src/comfy_memory.rs), so a library
// that asks the driver for memory in the middle of a denoising step can fail there, or stall every stream of the device
// while the driver serves it. For those callers the K-split form of the GEMM gets its scratch (per-chunk arrival
// counters, then int32 tile sums) from this array, which is part of the loaded module on every GPU until the process
// exits: 64 KiB of counters + 16 tiles x 256 x 256 x 4 B of sums = 4,259,840 bytes.
constexpr int kStaticMaxTiles = 16;
constexpr size_t kStaticCounterBytes = 1 << 16;
constexpr size_t kStaticScratchBytes = kStaticCounterBytes + (size_t)kStaticMaxTiles * 256 * 256 * sizeof(int);
static __device__ __align__(256) int g_static_scratch[kStaticScratchBytes / sizeof(int)];

// Device address of the array for the current device. In host code the array's name is only a handle for the runtime,
// not an address a kernel could use, so the address is looked up once per device and remembered.
int static_scratch_ptr(int dev, int** out) {
    static int* ptr[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    int*& p = ptr[dev & 63];
    if (!p) {
        void* addr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&addr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        p = reinterpret_cast<int*>(addr);
    }
    *out = p;
    return 0;
}

}  // namespace

// D[M,N] = out((A . W^T) * xs[m] * ws[n] + bias[n]) like gpu_int8_gemm, for problems of at most 16 output tiles
// (a few hundred rows or columns) with a long K, cut along K so that more SMs stream them. No cudaMalloc, cudaFree or
// other allocating call is made, now or later: the scratch is the static array above.
//   -205  the problem needs more than 16 tiles: beyond the array. Use gpu_int8_gemm.
// The first call on a device looks up the array's address (cudaGetSymbolAddress); make that call before any stream
// capture starts. Every call zeroes the part of the array it will use (an asynchronous memset on `stream`) because
// the array keeps whatever the previous call left; two calls that overlap on the GPU (different streams, no
// dependency) would share counters and sums and corrupt each other: serialise them.
GPU_API int gpu_int8_gemm_noalloc(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias,
                                  void* D, int64_t M, int64_t N, int64_t K, int out_dt, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (M == 0 || N == 0 || K == 0) return 0;
    if (out_dt < 0 || out_dt > 2) return -200;
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return -200;
    if ((K % 16) != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return -202;
    int dev = 0;
    cudaGetDevice(&dev);
    const int clusters = device_sm_count(dev) / 2;
    GemmParams p{};
    p.xs = xs, p.ws = ws, p.bias = bias, p.D = D;
    p.M = (int)M, p.N = (int)N, p.K = (int)K;
    const int esz = out_dt == DT_F32 ? 4 : 2;
    auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    p.vec_ok = (N % 8 == 0) && al16(D) && al16(ws) && al16(bias);
    p.tma_store = al16(D) && ((N * esz) % 16 == 0);
    p.ksub = K <= BK ? 1 : 2;
    p.k_iters = (int)((K + p.ksub * BK - 1) / (p.ksub * BK));
    // the width that fills the clusters best, widened while the tiles outnumber the array's 16 slots
    int bn = choose_bn(M, N, clusters);
    p.tiles_m = (int)((M + 2 * BM - 1) / (2 * BM));
    while (bn < 256 && p.tiles_m * ((N + bn - 1) / bn) > kStaticMaxTiles) bn += 32;
    p.bn = bn;
    p.idesc = umma_idesc_i8(2 * BM, bn);
    const int stage_bytes = p.ksub * (BM * BK + (bn / 2) * BK);
    const int stages = (kSmemBytes - 1024 - kTailBytes - kStagingBytes) / stage_bytes;
    p.stages = stages > kMaxStages ? kMaxStages : stages;
    p.tiles_n = (int)((N + bn - 1) / bn);
    p.num_tiles = p.tiles_m * p.tiles_n;
    if (p.num_tiles > kStaticMaxTiles) return -205;
    int splits = clusters / p.num_tiles;
    if (splits < 1) splits = 1;
    if (splits > p.k_iters) splits = p.k_iters;
    if (splits > 16) splits = 16;
    const int kps = (p.k_iters + splits - 1) / splits;
    splits = (p.k_iters + kps - 1) / kps;
    p.whole_tiles = p.num_tiles, p.splits = 0, p.kps = p.k_iters, p.num_items = p.num_tiles;
    if (splits >= 2) {
        int* scratch = nullptr;
        if (int rc = static_scratch_ptr(dev, &scratch)) return rc;
        const size_t used = kStaticCounterBytes + (size_t)p.num_tiles * kCountersPerSlot * 32 * 32 * sizeof(int);
        const cudaError_t e = cudaMemsetAsync(scratch, 0, used, st);
        if (e != cudaSuccess) return (int)e;
        p.scratch = scratch;
        p.partials = scratch + kStaticCounterBytes / sizeof(int);
        p.whole_tiles = 0, p.splits = splits, p.kps = kps, p.num_items = p.num_tiles * splits;
    }
    CUtensorMap ta, tw, td;
    if (!make_operand_tmap(&ta, A, M, K, BM) || !make_operand_tmap(&tw, W, N, K, bn / 2)) return -203;
    if (p.tma_store) {
        if (!make_output_tmap(&td, D, M, N, esz)) return -203;
    } else {
        td = ta;
    }
    const int grid = 2 * (p.num_items < clusters ? p.num_items : clusters);
    if (out_dt == DT_F32) return launch_pair<float, EPI_PLAIN>(ta, tw, td, p, grid, st);
    if (out_dt == DT_F16) return launch_pair<half, EPI_PLAIN>(ta, tw, td, p, grid, st);
    return launch_pair<bf16, EPI_PLAIN>(ta, tw, td, p, grid, st);
}


// New (tensor parallelism): the persistent GEMM normally takes every SM pair of the device, and a collective's kernels
// launched beside it on another stream then wait for it to end. A limit of n > 0 makes gpu_int8_gemm* launches that follow
// (any thread, any device of the process) occupy at most n CTA pairs, leaving the other SMs to concurrent kernels;
// 0 restores the default. Returns the previous limit.
GPU_API int gpu_int8_gemm_set_cluster_limit(int clusters) {
    return g_cluster_limit.exchange(clusters < 0 ? 0 : clusters, std::memory_order_relaxed);
}

// Reads and clears the device status word (synchronises the device). 0 = no kernel gave up a wait.
GPU_API int gpu_kernels_status(int* status) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_kernel_status, &zero, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    int qv = 0;
    if (int rc = quant_status_read_clear(&qv)) return rc;
    if (v) g_workspace_epoch.fetch_add(1, std::memory_order_acq_rel);   // scratch may hold partial sums: clear before reuse
    if (status) *status = v ? v : qv;
    return 0;
}
