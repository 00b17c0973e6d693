// Quantize-at-load weight packers and their inverses, plus the fp16 (SD/SDXL) row quantizer that serves both
// weights at load and activations at run time.
//
//   gpu_sd_quant_rows      fp16 rows -> [R64|R256] -> int8 + fp32 row scale          reference csrc/sd.cu:578-606
//   gpu_convrot_requant    f32/bf16 weight -> R256 -> int8 + row scale (seed 0: nearest-even; else PCG-hash
//                          stochastic rounding)                                       csrc/kernels.cu:1362-1389,1409-1420
//   gpu_convrot_dequant    int8 ConvRot weight -> original basis (f32/bf16)           csrc/kernels.cu:1345-1354,1393-1405
//   gpu_embed_dequant      int8 ConvRot embedding rows -> f32 rows of bf16 values     csrc/kernels.cu:622-638
//   gpu_dequant_i8         int8 * row scale -> f32                                    csrc/kernels.cu:330-343
//   gpu_w6_decode          6-bit two-plane codes + e4m3 group scales -> int8          csrc/h3.cu:11-46
//
// One CTA per row; the row lives in shared memory as fp32 (padded against bank conflicts). The rotation runs as
// two register phases: each thread takes 16 consecutive elements (index bits 0-3: radix-4 stages 0 and 1), then 16
// elements 16 apart (index bits 4-7: stages 2 and 3; groups of 64 have only stage 2), so a row is read and written
// in shared memory twice whatever its length. Every butterfly adds in the reference's left-to-right order.
#include <cstdlib>
#include <cuda_fp8.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "w6_decode.cuh"

// quant_rows.cu
GPU_API int gpu_quant_rows(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                           int64_t up_offset, const float* norm_w, float eps, const void* mod_scale, const void* mod_shift,
                           int8_t* q, float* scales, int M, int K, int rotate, void* stream);

namespace {

// element i of the row sits at word i + 4*(i/16): 16-element runs stay 16-byte aligned and consecutive runs start
// 20 banks apart
__device__ __forceinline__ int pad(int i) { return i + ((i >> 4) << 2); }
__host__ __device__ constexpr int padded_words(int K) { return K + ((K + 15) / 16) * 4 + 4; }

__device__ __forceinline__ void h4(float& x0, float& x1, float& x2, float& x3) {
    const float s = __fadd_rn(x0, x1), d = __fsub_rn(x0, x1);
    const float r0 = __fmul_rn(0.5f, __fsub_rn(__fadd_rn(s, x2), x3));
    const float r1 = __fmul_rn(0.5f, __fadd_rn(__fsub_rn(s, x2), x3));
    const float r2 = __fmul_rn(0.5f, __fadd_rn(__fadd_rn(d, x2), x3));
    const float r3 = __fmul_rn(0.5f, __fadd_rn(__fadd_rn(-d, x2), x3));
    x0 = r0, x1 = r1, x2 = r2, x3 = r3;
}

// In-place rotation of the padded shared-memory row: groups of 256 (four stages) or 64 (three).
__device__ void rotate_row_smem(float* row, int K, int group) {
    // phase 1: stages 0 and 1 on 16 consecutive elements
    for (int c = threadIdx.x; c < K / 16; c += blockDim.x) {
        float v[16];
        float* base = row + pad(c * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = reinterpret_cast<const float4*>(base)[i];
            v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
        }
#pragma unroll
        for (int i = 0; i < 16; i += 4) h4(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) h4(v[i], v[i + 4], v[i + 8], v[i + 12]);
#pragma unroll
        for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(base)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
    __syncthreads();
    if (group == 256) {
        // phase 2: stages 2 and 3 on elements e + 16 r of a 256-group
        for (int c = threadIdx.x; c < K / 16; c += blockDim.x) {
            const int g = c >> 4, e = c & 15;
            float v[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) v[r] = row[pad((g << 8) + e + 16 * r)];
#pragma unroll
            for (int i = 0; i < 16; i += 4) h4(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) h4(v[i], v[i + 4], v[i + 8], v[i + 12]);
#pragma unroll
            for (int r = 0; r < 16; ++r) row[pad((g << 8) + e + 16 * r)] = v[r];
        }
    } else {
        // phase 2: stage 2 on elements e + 16 r, r < 4, of a 64-group
        for (int c = threadIdx.x; c < K / 4; c += blockDim.x) {
            const int g = c >> 4, e = c & 15;
            float* b = row;
            const int i0 = (g << 6) + e;
            float x0 = b[pad(i0)], x1 = b[pad(i0 + 16)], x2 = b[pad(i0 + 32)], x3 = b[pad(i0 + 48)];
            h4(x0, x1, x2, x3);
            b[pad(i0)] = x0, b[pad(i0 + 16)] = x1, b[pad(i0 + 32)] = x2, b[pad(i0 + 48)] = x3;
        }
    }
    __syncthreads();
}

__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.f;
    return warp_max(t);
}

// block_sum of the reference (csrc/common.cuh:42-55): xor-shuffle tree over each warp, then over the warp sums
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
    return t;
}

// ---- fp16 row quantizer ---------------------------------------------------------------------------------
// rotation, row maximum, scale and codes of a row held in (padded) shared memory as fp32
__device__ void sd_quant_tail(float* row, float* red, int8_t* __restrict__ qr, float* __restrict__ scale_out, int K, int rotate,
                              int vec) {
    if (rotate) rotate_row_smem(row, K, rotate);
    float mx = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, fabsf(rnd<half>(row[pad(k)])));
    mx = block_max(mx, red);
    const float scale = __fdiv_rn(fmaxf(mx, 1e-30f), 127.f);
    if (threadIdx.x == 0) *scale_out = scale;
    const float sh = rnd<half>(scale);
    const float st = sh > 0.f ? sh : scale;  // a scale below half's range divides in float
    if (vec) {
        for (int c = threadIdx.x; c < K / 8; c += blockDim.x) {
            const float* s = row + pad(c * 8);
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int qi = clamp_rint_i8(rnd<half>(__fdiv_rn(rnd<half>(s[j]), st)), -128.f);
                w[j >> 2] |= (uint32_t)(qi & 0xff) << (8 * (j & 3));
            }
            reinterpret_cast<uint2*>(qr)[c] = make_uint2(w[0], w[1]);
        }
    } else {
        for (int k = threadIdx.x; k < K; k += blockDim.x)
            qr[k] = (int8_t)clamp_rint_i8(rnd<half>(__fdiv_rn(rnd<half>(row[pad(k)]), st)), -128.f);
    }
}

__global__ void __launch_bounds__(256) sd_quant_rows_kernel(const half* __restrict__ x, int64_t x_stride,
                                                            int8_t* __restrict__ q, float* __restrict__ scales, int K,
                                                            int rotate, int vec) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const int64_t m = blockIdx.x;
    const half* r = x + m * x_stride;
    if (vec) {
        for (int c = threadIdx.x; c < K / 8; c += blockDim.x) {
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(r) + c);
            const __half2* h = reinterpret_cast<const __half2*>(&u);
            float* d = row + pad(c * 8);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                d[2 * i] = f.x, d[2 * i + 1] = f.y;
            }
        }
    } else {
        for (int k = threadIdx.x; k < K; k += blockDim.x) row[pad(k)] = __half2float(r[k]);
    }
    __syncthreads();
    sd_quant_tail(row, red, q + m * (int64_t)K, scales + m, K, rotate, vec);
}

// The same quantizer for the run-time case (activations of every SD linear): rows in registers instead of shared memory.
// A thread holds 16 consecutive values: stages 0 and 1 of the rotation are its own; stage 2 (and 3 for groups of 256)
// pairs it with the three other lanes whose position differs in index bits 4-5 (6-7) through shuffles, each lane
// computing its own output row of the H4 block with the reference's association ((+-x0 +- x1) +- x2) +- x3. Several rows
// per CTA, row maximum through a shared-memory atomicMax. Bit-identical to the kernel above.
template <int ROT>
__global__ void __launch_bounds__(512) sd_quant_rows_reg_kernel(const half* __restrict__ x, int64_t x_stride,
                                                                int8_t* __restrict__ q, float* __restrict__ scales, int M, int K,
                                                                int tpr, int rows_per_cta) {
    extern __shared__ unsigned amax_s[];     // [rows_per_cta]
    for (int i = threadIdx.x; i < rows_per_cta; i += blockDim.x) amax_s[i] = 0u;
    __syncthreads();
    const int rloc = threadIdx.x / tpr, tin = threadIdx.x - rloc * tpr;
    const int64_t m_raw = (int64_t)blockIdx.x * rows_per_cta + rloc;
    const bool live = m_raw < M;
    const int64_t m = live ? m_raw : M - 1;      // idle rows recompute the last row and store nothing
    const half* r = x + m * x_stride + tin * 16;
    float v[16];
    {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(r)), b = __ldg(reinterpret_cast<const uint4*>(r) + 1);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x, v[2 * i + 1] = f.y;
        }
    }
    if (ROT) {
#pragma unroll
        for (int i = 0; i < 16; i += 4) h4(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) h4(v[i], v[i + 4], v[i + 8], v[i + 12]);
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int st = 0; st < (ROT == 256 ? 2 : 1); ++st) {
            const int sh = st ? 4 : 1;                    // lane distance between the block's four inputs
            const int pos = (tin / sh) & 3;               // this lane's row of the H4 block
            const int base = lane - pos * sh;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float x0 = __shfl_sync(0xffffffffu, v[i], base), x1 = __shfl_sync(0xffffffffu, v[i], base + sh);
                const float x2 = __shfl_sync(0xffffffffu, v[i], base + 2 * sh), x3 = __shfl_sync(0xffffffffu, v[i], base + 3 * sh);
                const float a = pos == 3 ? -x0 : x0, b = pos == 2 ? -x1 : x1, c = pos == 1 ? -x2 : x2, d = pos == 0 ? -x3 : x3;
                v[i] = __fmul_rn(0.5f, __fadd_rn(__fadd_rn(__fadd_rn(a, b), c), d));
            }
        }
    }
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = rnd<half>(v[i]), mx = fmaxf(mx, fabsf(v[i]));
    atomicMax(amax_s + rloc, __float_as_uint(mx));       // non-negative floats order as integers
    __syncthreads();
    mx = __uint_as_float(amax_s[rloc]);
    const float scale = __fdiv_rn(fmaxf(mx, 1e-30f), 127.f);
    if (live && tin == 0) scales[m] = scale;
    const float sh16 = rnd<half>(scale);
    const float st = sh16 > 0.f ? sh16 : scale;
    uint32_t o[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int qi = clamp_rint_i8(rnd<half>(__fdiv_rn(v[i], st)), -128.f);
        o[i >> 2] |= (uint32_t)(qi & 0xff) << (8 * (i & 3));
    }
    if (live) *reinterpret_cast<uint4*>(q + m * (int64_t)K + tin * 16) = make_uint4(o[0], o[1], o[2], o[3]);
}

// The same quantizer over a row that another of the reference's kernels would have written in half first
// (csrc/sd.cu:611-724): the row is computed as that kernel computes it, rounded to half, then quantized as above.
// 256 threads, each adding elements t, t + 256, ... and then the block tree: the reference's order of additions.
enum { SDQ_LN = 1, SDQ_GEGLU = 2, SDQ_UNPAD = 3, SDQ_GN = 4 };
struct SdSrc {
    const half* x;
    int64_t x_stride;   // LN: elements between rows
    const float* w;     // LN, GN: weight and bias
    const float* b;
    float eps;          // LN, GN
    int heads, d, dp;   // UNPAD: heads of d values stored dp wide
    const double* sums; // GN: per (image, group) sum and sum of squares
    int groups;         // GN
    int64_t P;          // GN: pixels per image
    double cnt;         // GN: values per group, P * C / groups
};

// GroupNorm statistics of x [N, P, C] half: per (image, group) the sum and the sum of squares, accumulated in double
// from per-block float sums as the reference's sd_group_sums_kernel forms them (csrc/sd.cu:209-233: 256 threads, thread
// t takes values t, t + 256, ... of the block's pixel range, then the block tree), so the statistics come out the same.
__global__ void __launch_bounds__(256) sd_group_sums_kernel(const half* __restrict__ x, double* __restrict__ sums, int64_t P,
                                                            int C, int G, int splits) {
    __shared__ float red[33];
    const int ng = blockIdx.x, split = blockIdx.y;
    const int n = ng / G, g = ng % G, per = C / G;
    const int64_t base = (int64_t)n * P * C + g * per;
    const int64_t p0 = P * split / splits, p1 = P * (split + 1) / splits;
    const int64_t count = (p1 - p0) * per;
    float s = 0.f, ss = 0.f;
    for (int64_t i = threadIdx.x; i < count; i += blockDim.x) {
        const float v = __half2float(x[base + (p0 + i / per) * C + (int)(i % per)]);
        s = __fadd_rn(s, v);
        ss = __fmaf_rn(v, v, ss);
    }
    s = block_sum(s, red);
    __syncthreads();
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) {
        atomicAdd(&sums[ng * 2], (double)s);
        atomicAdd(&sums[ng * 2 + 1], (double)ss);
    }
}
template <int MODE>
__global__ void __launch_bounds__(256) sd_quant_src_kernel(const SdSrc p, int8_t* __restrict__ q, float* __restrict__ scales,
                                                           int K, int rotate, int vec) {
    extern __shared__ float row[];
    __shared__ float red[33];
    const int64_t m = blockIdx.x;
    if (MODE == SDQ_LN) {            // sd_layer_norm_kernel, csrc/sd.cu:312-328
        const half* r = p.x + m * p.x_stride;
        float s = 0.f;
        for (int k = threadIdx.x; k < K; k += blockDim.x) s = __fadd_rn(s, __half2float(r[k]));
        const float mean = __fdiv_rn(block_sum(s, red), (float)K);
        float ss = 0.f;
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
            const float d = __fsub_rn(__half2float(r[k]), mean);
            ss = __fmaf_rn(d, d, ss);
        }
        const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(block_sum(ss, red), (float)K), p.eps));
        for (int k = threadIdx.x; k < K; k += blockDim.x)
            row[pad(k)] = rnd<half>(__fmaf_rn(__fmul_rn(__fsub_rn(__half2float(r[k]), mean), rstd), p.w[k], p.b[k]));
    } else if (MODE == SDQ_GEGLU) {  // sd_geglu_kernel: [M, 2K], value then gate
        const half* r = p.x + m * 2 * (int64_t)K;
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
            const float g = rnd<half>(gelu_f(__half2float(r[K + k])));
            row[pad(k)] = rnd<half>(__fmul_rn(__half2float(r[k]), g));
        }
    } else if (MODE == SDQ_UNPAD) {  // sd_unpad_heads
        const half* r = p.x + m * (int64_t)p.heads * p.dp;
        for (int k = threadIdx.x; k < K; k += blockDim.x) row[pad(k)] = __half2float(r[(k / p.d) * p.dp + k % p.d]);
    } else {                         // sd_group_apply_kernel without SiLU: row m is a pixel of image m / P (csrc/sd.cu:198-205,244-255)
        __shared__ float2 stat[256];
        const int n = (int)(m / p.P);
        for (int g = threadIdx.x; g < p.groups; g += blockDim.x) {
            const double su = p.sums[(n * p.groups + g) * 2], sq = p.sums[(n * p.groups + g) * 2 + 1];
            const double mean = su / p.cnt;
            const double var = fmax(fma(-mean, mean, sq / p.cnt), 0.0);
            stat[g] = make_float2((float)mean, (float)(1.0 / sqrt(var + (double)p.eps)));
        }
        __syncthreads();
        const half* r = p.x + m * (int64_t)K;
        const int per = K / p.groups;
        for (int c = threadIdx.x; c < K; c += blockDim.x) {
            const float2 st = stat[c / per];
            row[pad(c)] = rnd<half>(__fmaf_rn(__fmul_rn(__fsub_rn(__half2float(r[c]), st.x), st.y), p.w[c], p.b[c]));
        }
    }
    __syncthreads();
    sd_quant_tail(row, red, q + m * (int64_t)K, scales + m, K, rotate, vec);
}

// ---- ConvRot weight requant / dequant -------------------------------------------------------------------
__device__ __forceinline__ uint32_t pcg_hash(uint32_t x) {
    const uint32_t state = x * 747796405u + 2891336453u;
    const uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
    return (word >> 22u) ^ word;
}
__device__ __forceinline__ float noisy_sum(float scaled, float noise, float*) { return __fadd_rn(scaled, noise); }
__device__ __forceinline__ float noisy_sum(float scaled, float noise, bf16*) {
    return __bfloat162float(__hadd(__float2bfloat16_rn(scaled), __float2bfloat16_rn(noise)));
}
template <typename T> __device__ __forceinline__ float finite_max_t();
template <> __device__ __forceinline__ float finite_max_t<float>() { return FLT_MAX; }
template <> __device__ __forceinline__ float finite_max_t<bf16>() { return 3.38953139e38f; }

template <typename T>
__global__ void __launch_bounds__(512) convrot_requant_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                                                              float* __restrict__ scales, int K, uint64_t seed) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const int64_t m = blockIdx.x;
    const T* r = x + m * (int64_t)K;
    for (int k = threadIdx.x; k < K; k += blockDim.x) row[pad(k)] = to_f<T>(r[k]);
    __syncthreads();
    rotate_row_smem(row, K, 256);
    float amax = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(row[pad(k)]));
    amax = block_max(amax, red);
    const float scale = fmaxf(fminf(amax, finite_max_t<T>()) * (1.f / 127.f), 1.0e-30f);
    if (threadIdx.x == 0) scales[m] = scale;
    const float st = rnd<T>(scale);
    for (int c = threadIdx.x; c < K / 4; c += blockDim.x) {
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = c * 4 + j;
            const float scaled = rnd<T>(__fdiv_rn(rnd<T>(row[pad(k)]), st));
            int qi;
            if (seed == 0) {
                qi = clamp_rint_i8(scaled, -128.f);
            } else {
                const uint64_t key = (uint64_t)(m * K + k) + seed;
                const uint32_t folded = (uint32_t)key ^ (uint32_t)(key >> 32);
                const float v = floorf(noisy_sum(scaled, (float)(pcg_hash(folded) >> 8) * 0x1.0p-24f, (T*)nullptr));
                qi = (int)fminf(127.f, fmaxf(-128.f, v));
            }
            w |= (uint32_t)(qi & 0xff) << (8 * j);
        }
        reinterpret_cast<uint32_t*>(q + m * (int64_t)K)[c] = w;
    }
}

// OUT_BF16_IN_F32: embed_dequant writes f32 rows holding bf16-rounded values
template <typename T, bool ROUND_BF16>
__global__ void __launch_bounds__(512) convrot_dequant_kernel(const int8_t* __restrict__ q, const float* __restrict__ s,
                                                              T* __restrict__ out, int K) {
    extern __shared__ float row[];
    const int64_t m = blockIdx.x;
    const float sc = s[m];
    for (int c = threadIdx.x; c < K / 4; c += blockDim.x) {
        const char4 v = reinterpret_cast<const char4*>(q + m * (int64_t)K)[c];
        float* d = row + pad(c * 4);
        d[0] = __fmul_rn((float)v.x, sc), d[1] = __fmul_rn((float)v.y, sc);
        d[2] = __fmul_rn((float)v.z, sc), d[3] = __fmul_rn((float)v.w, sc);
    }
    __syncthreads();
    rotate_row_smem(row, K, 256);
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = row[pad(k)];
        out[m * (int64_t)K + k] = from_f<T>(ROUND_BF16 ? rnd<bf16>(v) : v);
    }
}

__global__ void dequant_i8_kernel(const int8_t* __restrict__ q, const float* __restrict__ s, float* __restrict__ out,
                                  int64_t N, int64_t K) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= N * K) return;
    const char4 v = *reinterpret_cast<const char4*>(q + i);
    const float sc = s[i / K];
    *reinterpret_cast<float4*>(out + i) =
        make_float4(__fmul_rn(v.x, sc), __fmul_rn(v.y, sc), __fmul_rn(v.z, sc), __fmul_rn(v.w, sc));
}

// ---- W6 decode ------------------------------------------------------------------------------------------
__device__ __forceinline__ float e4m3_to_f(uint8_t v) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3)));
}
// One thread decodes 16 consecutive codes: 8 nibble bytes, 4 top-bit bytes, one group scale (G % 16 == 0).
__global__ void __launch_bounds__(256) w6_decode_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ s_rel,
                                                        int8_t* __restrict__ out, int64_t N, int K, int G) {
    const int64_t per = K / 16;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * per) return;
    const int64_t n = i / per;
    const int c = (int)(i - n * per);
    const uint8_t* row = q + n * (int64_t)(K / 4 * 3);
    const uint2 lo = __ldg(reinterpret_cast<const uint2*>(row + c * 8));
    const uint32_t hi = __ldg(reinterpret_cast<const uint32_t*>(row + K / 2 + c * 4));
    const float sc = e4m3_to_f(s_rel[n * (K / G) + c * 16 / G]);
    const uint32_t lw[2] = {lo.x, lo.y};
    uint32_t o[4];
#pragma unroll
    for (int e4 = 0; e4 < 4; ++e4) {  // four output words of four codes
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = e4 * 4 + j;  // code index 0..15
            const uint32_t nib = (lw[e >> 3] >> (4 * (e & 7))) & 15u;
            const uint32_t top = (hi >> (2 * e)) & 3u;
            const float cv = (float)(int)(nib | (top << 4)) - 32.f;
            const int d = (int)fminf(127.f, fmaxf(-127.f, nearbyintf(__fmul_rn(cv, sc))));
            w |= (uint32_t)(d & 0xff) << (8 * j);
        }
        o[e4] = w;
    }
    *reinterpret_cast<uint4*>(out + n * (int64_t)K + c * 16) = make_uint4(o[0], o[1], o[2], o[3]);
}

// ---- W6A8 packer: bf16 weight -> R256 -> 6-bit codes + e4m3 group scales + f32 channel scale -----------------------
// The algorithm of the reference's gpu_w6_requant (csrc/vendor/w6a8_requant.cu:59-154), per row:
//   rotate, round to bf16; per group of 32: step gs = amax / 31, refined by two least-squares rounds
//   (q = clamp(rint(w / gs), +-31); gs = sum(w q) / sum(q q)); channel scale sc = max |q gs| / 127;
//   s_rel = e4m3(gs / sc); every element t = w / sc takes one of the 63 levels clamp(rint((i - 31) s_rel), +-127) that
//   bracket it, drawn with probability proportional to the distance (hash-keyed uniform), and is stored as i + 1.
// One thread per group (the sums are sequential over the group's 32 values, as there); maxima are order-free.
__device__ __forceinline__ float w6_level(int i, float s) {
    return fminf(127.f, fmaxf(-127.f, nearbyintf(__fmul_rn((float)(i - 31), s))));
}
__device__ __forceinline__ int w6_first_level_not_below(float t, float s, float inv_s) {
    int i = __float2int_rn(__fmul_rn(__fsub_rn(ceilf(t), 0.5f), inv_s)) + 31;
    i = min(max(i, 0), 63);
    while (i > 0 && w6_level(i - 1, s) >= t) --i;
    while (i < 63 && w6_level(i, s) < t) ++i;
    return i;
}
__global__ void __launch_bounds__(256) w6_requant_kernel(const bf16* __restrict__ w, uint8_t* __restrict__ packed,
                                                         uint8_t* __restrict__ s_rel, float* __restrict__ s_channel, int K,
                                                         uint64_t seed) {
    extern __shared__ float row[];            // padded row, then K / 32 group steps
    __shared__ float red[32];
    float* gstep = row + padded_words(K);
    const int64_t n = blockIdx.x;
    const bf16* r = w + n * (int64_t)K;
    for (int k = threadIdx.x; k < K; k += blockDim.x) row[pad(k)] = __bfloat162float(r[k]);
    __syncthreads();
    rotate_row_smem(row, K, 256);
    for (int k = threadIdx.x; k < K; k += blockDim.x) row[pad(k)] = rnd<bf16>(row[pad(k)]);   // the rotated weight lives in bf16
    __syncthreads();
    const int groups = K / 32;
    float amax_row = 0.f;
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        float v[32];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = row[pad(g * 32 + i)], amax = fmaxf(amax, fabsf(v[i]));
        float gs = fmaxf(__fdiv_rn(amax, 31.f), 1e-8f);
        float inv = __fdiv_rn(1.f, gs);
#pragma unroll 1
        for (int it = 0; it < 2; ++it) {
            float num = 0.f, den = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float q = fminf(31.f, fmaxf(-31.f, nearbyintf(__fmul_rn(v[i], inv))));
                num = __fmaf_rn(v[i], q, num);
                den = __fmaf_rn(q, q, den);
            }
            gs = fmaxf(__fdiv_rn(num, fmaxf(den, 1e-8f)), 1e-8f);
            inv = __fdiv_rn(1.f, gs);
        }
        gstep[g] = gs;
#pragma unroll
        for (int i = 0; i < 32; ++i)
            amax_row = fmaxf(amax_row, fabsf(__fmul_rn(fminf(31.f, fmaxf(-31.f, nearbyintf(__fmul_rn(v[i], inv)))), gs)));
    }
    amax_row = block_max(amax_row, red);
    const float sc = fmaxf(__fdiv_rn(amax_row, 127.f), 1e-8f);
    const float inv_sc = __fdiv_rn(1.f, sc);
    if (threadIdx.x == 0) s_channel[n] = sc;
    uint8_t* prow = packed + n * (int64_t)(K / 4 * 3);
    const uint32_t key = (uint32_t)seed ^ (uint32_t)(seed >> 32);
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        const uint8_t sb = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(gstep[g], sc), __NV_SATFINITE, __NV_E4M3);
        s_rel[n * groups + g] = sb;
        const float s = e4m3_to_f(sb);
        const float inv_s = __fdiv_rn(1.f, fmaxf(s, 1e-30f));
        uint32_t lo[4] = {0u, 0u, 0u, 0u}, hi[2] = {0u, 0u};
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
            const float t = __fmul_rn(row[pad(g * 32 + i)], inv_sc);
            const int pos = w6_first_level_not_below(t, s, inv_s);
            const int l = min(max(pos - 1, 0), 61);
            const float level_lo = w6_level(l, s);
            const uint32_t h = pcg_hash((uint32_t)(n * (int64_t)K + g * 32 + i) ^ key);
            const float u = __fmul_rn((float)(h >> 8), 1.0f / 16777216.0f);
            const float thr = __fmaf_rn(u, __fsub_rn(w6_level(l + 1, s), level_lo), level_lo);
            const uint32_t code = (uint32_t)min(l + (t > thr ? 1 : 0), 62) + 1u;
            lo[i >> 3] |= (code & 15u) << (4 * (i & 7));
            hi[i >> 4] |= ((code >> 4) & 3u) << (2 * (i & 15));
        }
        *reinterpret_cast<uint4*>(prow + g * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint2*>(prow + K / 2 + g * 8) = make_uint2(hi[0], hi[1]);
    }
}

// The same with 32 codes (one whole scale group when G is a multiple of 32) per thread and the permute-table decode of
// w6_decode.cuh: 16 + 8 bytes in, 32 bytes out per thread. The decode form is voted per warp, so every lane takes part
// (lanes past the end redo the last piece and store nothing).
__global__ void __launch_bounds__(256) w6_decode32_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ s_rel,
                                                          int8_t* __restrict__ out, int64_t N, int K, int G) {
    const int64_t per = K / 32;
    const int64_t total = N * per;
    const int64_t i_raw = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = i_raw < total;
    const int64_t i = live ? i_raw : total - 1;
    const int64_t n = i / per;
    const int c = (int)(i - n * per);
    const uint8_t* row = q + n * (int64_t)(K / 4 * 3);
    const uint4 lo = __ldg(reinterpret_cast<const uint4*>(row + c * 16));
    const uint2 hi = __ldg(reinterpret_cast<const uint2*>(row + K / 2 + c * 8));
    const uint32_t sb = s_rel[n * (K / G) + c * 32 / G];
    uint32_t o[8];
    w6_group(lo, hi.x, hi.y, sb, o);
    if (live) {
        uint4* d = reinterpret_cast<uint4*>(out + n * (int64_t)K + c * 32);
        d[0] = make_uint4(o[0], o[1], o[2], o[3]);
        d[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

int set_smem(const void* fn, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return e == cudaSuccess ? 0 : (int)e;
}
int row_threads(int work_items, int cap) {
    int t = (work_items + 31) / 32 * 32;
    return t < 32 ? 32 : (t > cap ? cap : t);
}

}  // namespace

// x fp16 [M, K] (row pitch x_stride elements) -> q int8 [M, K], scales f32 [M]; rotate 0, 64 or 256 (must divide K).
GPU_API int gpu_sd_quant_rows(const void* x, int64_t x_stride, int8_t* q, float* scales, int M, int K, int rotate,
                              void* stream) {
    if ((rotate != 0 && rotate != 64 && rotate != 256) || (rotate && K % rotate)) return -1;
    if (M <= 0 || K <= 0) return 0;
    {   // rows of whole 32-value pieces: the quantizer's register kernel (transposition through shared memory for R256)
        int rc = 0;
        if (sd_quant_rows_fast(x, x_stride, q, scales, M, K, rotate, (cudaStream_t)stream, &rc)) return rc;
    }
    // register kernel: whole 16-value pieces per thread, rotation groups inside a warp, aligned rows
    const int tpr = K / 16;
    if (K % 16 == 0 && tpr <= 512 && x_stride % 8 == 0 && (((uintptr_t)x & 15) == 0) && (((uintptr_t)q & 15) == 0)) {
        const int gcd32 = tpr % 32 == 0 ? 32 : tpr % 16 == 0 ? 16 : tpr % 8 == 0 ? 8 : tpr % 4 == 0 ? 4 : tpr % 2 == 0 ? 2 : 1;
        const int r0 = 32 / gcd32;                       // rows that make the CTA a whole number of warps
        int rows = r0 * (256 / (tpr * r0) > 0 ? 256 / (tpr * r0) : 1);
        if (rows * tpr <= 512) {
            const int grid = (M + rows - 1) / rows, threads = rows * tpr;
            const size_t sm = (size_t)rows * sizeof(unsigned);
            cudaStream_t st = (cudaStream_t)stream;
            const half* xh = (const half*)x;
            if (rotate == 0) sd_quant_rows_reg_kernel<0><<<grid, threads, sm, st>>>(xh, x_stride, q, scales, M, K, tpr, rows);
            else if (rotate == 64) sd_quant_rows_reg_kernel<64><<<grid, threads, sm, st>>>(xh, x_stride, q, scales, M, K, tpr, rows);
            else sd_quant_rows_reg_kernel<256><<<grid, threads, sm, st>>>(xh, x_stride, q, scales, M, K, tpr, rows);
            KCHECK();
            return 0;
        }
    }
    const size_t smem = (size_t)padded_words(K) * sizeof(float);
    if (int rc = set_smem((const void*)sd_quant_rows_kernel, smem)) return rc;
    const int vec = (K % 8 == 0) && (x_stride % 8 == 0) && (((uintptr_t)x & 15) == 0) && (((uintptr_t)q & 7) == 0);
    sd_quant_rows_kernel<<<M, row_threads(K / 8, 256), smem, (cudaStream_t)stream>>>((const half*)x, x_stride, q, scales, K,
                                                                                     rotate, vec);
    KCHECK();
    return 0;
}

namespace {
template <int MODE>
int launch_sd_src(const SdSrc& p, int8_t* q, float* scales, int M, int K, int rotate, cudaStream_t st) {
    if ((rotate != 0 && rotate != 64 && rotate != 256) || (rotate && K % rotate)) return -1;
    if (M <= 0 || K <= 0) return 0;
    const size_t smem = (size_t)padded_words(K) * sizeof(float);
    if (int rc = set_smem((const void*)sd_quant_src_kernel<MODE>, smem)) return rc;
    const int vec = (K % 8 == 0) && (((uintptr_t)q & 7) == 0);
    sd_quant_src_kernel<MODE><<<M, 256, smem, st>>>(p, q, scales, K, rotate, vec);
    KCHECK();
    return 0;
}
}  // namespace

// LayerNorm of half rows (f32 weight and bias) fused into the quantizer: gpu_sd_layer_norm then gpu_sd_quant_rows,
// without the half intermediate in memory. csrc/sd.cu:690-696.
GPU_API int gpu_sd_ln_quant_rows(const void* x, int64_t x_stride, const float* w, const float* b, float eps, int8_t* q,
                                 float* scales, int M, int K, int rotate, void* stream) {
    SdSrc p{(const half*)x, x_stride, w, b, eps, 0, 0, 0, nullptr, 0, 0, 0.0};
    return launch_sd_src<SDQ_LN>(p, q, scales, M, K, rotate, (cudaStream_t)stream);
}
// GEGLU of in [M, 2 I] (value then gate) fused into the quantizer of the [M, I] result. csrc/sd.cu:697-702.
GPU_API int gpu_sd_geglu_quant_rows(const void* in, int8_t* q, float* scales, int M, int I, int rotate, void* stream) {
    SdSrc p{(const half*)in, 0, nullptr, nullptr, 0.f, 0, 0, 0, nullptr, 0, 0, 0.0};
    return launch_sd_src<SDQ_GEGLU>(p, q, scales, M, I, rotate, (cudaStream_t)stream);
}
// Head un-padding of src [M, H, dp] fused into the quantizer of the [M, H * d] result. csrc/sd.cu:703-708.
GPU_API int gpu_sd_unpad_quant_rows(const void* src, int8_t* q, float* scales, int M, int H, int d, int dp, int rotate,
                                    void* stream) {
    SdSrc p{(const half*)src, 0, nullptr, nullptr, 0.f, H, d, dp, nullptr, 0, 0, 0.0};
    return launch_sd_src<SDQ_UNPAD>(p, q, scales, M, H * d, rotate, (cudaStream_t)stream);
}

// GroupNorm (no SiLU) of x [N, P, C] half fused into the quantizer of its [N * P, C] rows. `sums` is scratch of
// N * G * 2 doubles + 16 bytes, as the reference's gpu_sd_group_norm takes it; it is cleared here and holds the groups'
// sums afterwards (the reference overwrites the first half of each pair with (mean, rstd) as floats; nothing reads
// them after the call). -1: C % G, G > 256 or a bad rotate. csrc/sd.cu:710-724.
GPU_API int gpu_sd_group_norm_quant_rows(const void* x, const float* w, const float* b, void* sums, int N, int64_t P, int C,
                                         int G, float eps, int8_t* q, float* scales, int rotate, void* stream) {
    if (G <= 0 || C % G || G > 256) return -1;
    if ((rotate != 0 && rotate != 64 && rotate != 256) || (rotate && C % rotate)) return -1;
    if (N <= 0 || P <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const cudaError_t e = cudaMemsetAsync(sums, 0, (size_t)N * G * 2 * sizeof(double) + 16, st);
    if (e != cudaSuccess) return (int)e;
    const int64_t want = P * (C / G) / 4096;
    const int splits = want < 1 ? 1 : want > 64 ? 64 : (int)want;
    sd_group_sums_kernel<<<dim3(N * G, splits), 256, 0, st>>>((const half*)x, (double*)sums, P, C, G, splits);
    KCHECK();
    SdSrc p{(const half*)x, 0, w, b, eps, 0, 0, 0, (const double*)sums, G, P, (double)P * (C / G)};
    return launch_sd_src<SDQ_GN>(p, q, scales, (int)(N * P), C, rotate, st);
}

// x [N, K] f32 or bf16 in its original basis -> rotated q [N, K] int8 and row scales s [N].
GPU_API int gpu_convrot_requant(int dtype, const void* x, void* q, void* s, int64_t N, int K, uint64_t seed, void* stream) {
    if (K % 256) return -1;
    if (N <= 0) return 0;
    if (dtype != DT_F32 && dtype != DT_BF16) return -4;
    // Round-to-nearest packing (seed 0) is, operation for operation, the activation quantizer with no prologue and the
    // rotation on (the reference's two kernels share the scale rule and the rounding points, csrc/kernels.cu:241-255 and
    // :1372-1383), so it runs on that kernel, which keeps the row in registers: 12288 x 3072 f32 in a third of the time of
    // the shared-memory kernel below (which stays for the stochastic rounding and for rows the quantizer does not take).
    if (seed == 0 && K <= 32768 && N <= INT32_MAX && ((((uintptr_t)x | (uintptr_t)q) & 15) == 0))
        return gpu_quant_rows(dtype, 0, x, K, nullptr, 0, 0, nullptr, 0.f, nullptr, nullptr, (int8_t*)q, (float*)s, (int)N, K, 1, stream);
    const size_t smem = (size_t)padded_words(K) * sizeof(float);
    const int threads = row_threads(K / 16, 512);
    if (dtype == DT_F32) {
        if (int rc = set_smem((const void*)convrot_requant_kernel<float>, smem)) return rc;
        convrot_requant_kernel<float><<<(unsigned)N, threads, smem, (cudaStream_t)stream>>>((const float*)x, (int8_t*)q, (float*)s, K, seed);
    } else if (dtype == DT_BF16) {
        if (int rc = set_smem((const void*)convrot_requant_kernel<bf16>, smem)) return rc;
        convrot_requant_kernel<bf16><<<(unsigned)N, threads, smem, (cudaStream_t)stream>>>((const bf16*)x, (int8_t*)q, (float*)s, K, seed);
    } else {
        return -4;
    }
    KCHECK();
    return 0;
}

// q [N, K] int8 ConvRot weight, s [N] -> out [N, K] f32 or bf16 in the original basis.
GPU_API int gpu_convrot_dequant(int dtype, const void* q, const void* s, void* out, int64_t N, int K, void* stream) {
    if (K % 256) return -1;
    if (N <= 0) return 0;
    const size_t smem = (size_t)padded_words(K) * sizeof(float);
    const int threads = row_threads(K / 16, 512);
    if (dtype == DT_F32) {
        if (int rc = set_smem((const void*)convrot_dequant_kernel<float, false>, smem)) return rc;
        convrot_dequant_kernel<float, false><<<(unsigned)N, threads, smem, (cudaStream_t)stream>>>((const int8_t*)q, (const float*)s, (float*)out, K);
    } else if (dtype == DT_BF16) {
        if (int rc = set_smem((const void*)convrot_dequant_kernel<bf16, false>, smem)) return rc;
        convrot_dequant_kernel<bf16, false><<<(unsigned)N, threads, smem, (cudaStream_t)stream>>>((const int8_t*)q, (const float*)s, (bf16*)out, K);
    } else {
        return -4;
    }
    KCHECK();
    return 0;
}

// q [M, K] int8 ConvRot embedding rows, s [M] -> out f32 [M, K] holding bf16-rounded values; rotate must be set.
GPU_API int gpu_embed_dequant(const int8_t* q, const float* s, float* out, int M, int K, int rotate, void* stream) {
    if (!rotate || K % 256) return -1;
    if (M <= 0) return 0;
    const size_t smem = (size_t)padded_words(K) * sizeof(float);
    if (int rc = set_smem((const void*)convrot_dequant_kernel<float, true>, smem)) return rc;
    convrot_dequant_kernel<float, true><<<M, row_threads(K / 16, 512), smem, (cudaStream_t)stream>>>(q, s, out, K);
    KCHECK();
    return 0;
}

// out[n, k] = q[n, k] * s[n], f32.
GPU_API int gpu_dequant_i8(const int8_t* q, const float* s, float* out, int64_t N, int64_t K, void* stream) {
    if (K % 4) return -1;
    const int64_t n4 = N * K / 4;
    if (n4 <= 0) return 0;
    dequant_i8_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(q, s, out, N, K);
    KCHECK();
    return 0;
}

// q [N, 3K/4] (per row: K/2 nibble bytes, then K/4 bytes of top bits), s_rel [N, K/G] e4m3 -> out int8 [N, K]:
// out = clamp(rint((code - 32) * s_rel), +-127). K % 32 == 0 and G % 16 == 0, as the reference requires.
GPU_API int gpu_w6_decode(const void* q, const void* s_rel, void* out, int64_t N, int K, int G, void* stream) {
    if (K % 32 || G % 16) return -1;
    if (N <= 0 || K <= 0) return 0;
    // rows of 3K/4 bytes keep the 16-byte pieces of the nibble plane aligned when K % 64 == 0 (8-byte pieces of the other plane too)
    if (G % 32 == 0 && K % 64 == 0 && (((uintptr_t)q | (uintptr_t)out) & 15) == 0) {
        const int64_t n32 = N * (K / 32);
        w6_decode32_kernel<<<(unsigned)((n32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)q, (const uint8_t*)s_rel,
                                                                                          (int8_t*)out, N, K, G);
        KCHECK();
        return 0;
    }
    const int64_t n = N * (K / 16);
    w6_decode_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)q, (const uint8_t*)s_rel,
                                                                                 (int8_t*)out, N, K, G);
    KCHECK();
    return 0;
}

// bf16 weight [N, K] -> W6A8 storage: packed [N, 3K/4], s_rel e4m3 [N, K/32], s_channel f32 [N]; stochastic rounding keyed
// by `seed` and the element index. Replaces csrc/vendor/w6a8_requant.cu:246-257 (src/ffi.rs:132). -1: K % 256.
GPU_API int gpu_w6_requant(const void* weight, void* packed, void* s_rel, void* s_channel, int64_t N, int K, uint64_t seed,
                           void* stream) {
    if (K % 256) return -1;
    if (N <= 0) return 0;
    const size_t smem = (size_t)(padded_words(K) + K / 32) * sizeof(float);
    if (int rc = set_smem((const void*)w6_requant_kernel, smem)) return rc;
    w6_requant_kernel<<<(unsigned)N, 256, smem, (cudaStream_t)stream>>>((const bf16*)weight, (uint8_t*)packed, (uint8_t*)s_rel,
                                                                       (float*)s_channel, K, seed);
    KCHECK();
    return 0;
}

// The reference's Rust side imports this Windows (DXCore) video-memory budget query unconditionally
// (src/cuda.rs:136-153); non-zero means "no budget known", which is the answer everywhere else.
GPU_API int gpu_wddm_budget(uint64_t* budget, uint64_t* usage) {
    if (budget) *budget = 0;
    if (usage) *usage = 0;
    return 1;
}
