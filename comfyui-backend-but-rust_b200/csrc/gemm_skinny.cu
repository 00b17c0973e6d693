// int8 GEMM for a handful of rows (M <= 8): the adaLN-modulation and pooled-conditioning linears of the DiTs
// (M = 1 or 3 in the reference's src/anima.rs:733-737), where the work is streaming the weight matrix once.
// Bound by HBM, so it runs on the CUDA cores: A (a few KB) sits in shared memory, every warp streams four weight
// rows at a time with 16-byte loads, multiplies with dp4a into int32 (exact, like the tensor path), reduces across
// the warp and applies the same epilogue arithmetic as the tensor-core kernel.
#include "common.cuh"
#include "epilogue.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 4;

template <typename OutT, int EPI, int MT>
__global__ void __launch_bounds__(kWarps * 32) skinny_gemm_kernel(const SkinnyParams p) {
    extern __shared__ __align__(16) int8_t a_s[];   // [M][K]
    const int K = p.K;
    for (int i = threadIdx.x; i < p.M * K / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(a_s)[i] = __ldg(reinterpret_cast<const uint4*>(p.A) + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblocks = (p.N + kRowsPerWarp - 1) / kRowsPerWarp;
    for (int nb = blockIdx.x * kWarps + warp; nb < nblocks; nb += gridDim.x * kWarps) {
        const int n0 = nb * kRowsPerWarp;
        int acc[kRowsPerWarp][MT];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0;
        // several 512-byte K steps of the four rows are requested before the first is consumed: twelve to twenty-four
        // 16-byte loads in flight per lane instead of four
        constexpr int kAhead = MT <= 2 ? 6 : 3;      // one or two rows of A leave registers for twice the loads
        for (int kb = lane * 16; kb < K; kb += 512 * kAhead) {
            uint4 w[kAhead][kRowsPerWarp];
#pragma unroll
            for (int u = 0; u < kAhead; ++u)
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r) {
                    const int n = min(n0 + r, p.N - 1);   // rows past N repeat the last row; their results are dropped
                    const int k0 = kb + 512 * u;
                    w[u][r] = k0 < K ? __ldg(reinterpret_cast<const uint4*>(p.W + (int64_t)n * K + k0)) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int k0 = kb + 512 * u;
                if (k0 >= K) break;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m >= p.M) break;
                    const uint4 a = *reinterpret_cast<const uint4*>(a_s + m * K + k0);
#pragma unroll
                    for (int r = 0; r < kRowsPerWarp; ++r) {
                        int s = acc[r][m];
                        s = __dp4a((int)a.x, (int)w[u][r].x, s);
                        s = __dp4a((int)a.y, (int)w[u][r].y, s);
                        s = __dp4a((int)a.z, (int)w[u][r].z, s);
                        s = __dp4a((int)a.w, (int)w[u][r].w, s);
                        acc[r][m] = s;
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                int s = acc[r][m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                acc[r][m] = s;
            }
        // lane (r, m) = lane index r * MT + m finishes output (m, n0 + r)
        if (lane < kRowsPerWarp * MT) {
            const int r = lane / MT, m = lane % MT;
            const int n = n0 + r;
            int s = 0;
#pragma unroll
            for (int rr = 0; rr < kRowsPerWarp; ++rr)
#pragma unroll
                for (int mm = 0; mm < MT; ++mm)
                    if (rr == r && mm == m) s = acc[rr][mm];
            if (n < p.N && m < p.M) {
                const int64_t o = (int64_t)m * p.N + n;
                if (EPI == EPI_ACC) reinterpret_cast<int32_t*>(p.D)[o] = s;
                else {
                    const float bias = p.bias ? to_f<OutT>(reinterpret_cast<const OutT*>(p.bias)[n]) : 0.f;
                    const float rs = EPI == EPI_RESID ? to_f<OutT>(reinterpret_cast<const OutT*>(p.rscale)[n]) : 0.f;
                    const float rr = EPI == EPI_RESID ? to_f<OutT>(reinterpret_cast<const OutT*>(p.resid)[o]) : 0.f;
                    reinterpret_cast<OutT*>(p.D)[o] = from_f<OutT>(epilogue1<OutT, EPI>(s, p.xs[m], p.ws[n], bias, rs, rr, p.act));
                }
            }
        }
    }
}

template <typename OutT, int EPI>
int launch_mt(const SkinnyParams& p, int grid, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(skinny_gemm_kernel<OutT, EPI, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(skinny_gemm_kernel<OutT, EPI, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(skinny_gemm_kernel<OutT, EPI, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(skinny_gemm_kernel<OutT, EPI, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    if (p.M == 1) skinny_gemm_kernel<OutT, EPI, 1><<<grid, kWarps * 32, smem, st>>>(p);
    else if (p.M == 2) skinny_gemm_kernel<OutT, EPI, 2><<<grid, kWarps * 32, smem, st>>>(p);
    else if (p.M <= 4) skinny_gemm_kernel<OutT, EPI, 4><<<grid, kWarps * 32, smem, st>>>(p);
    else skinny_gemm_kernel<OutT, EPI, 8><<<grid, kWarps * 32, smem, st>>>(p);
    KCHECK();
    return 0;
}

template <typename OutT>
int launch_epi(int epi, const SkinnyParams& p, int grid, size_t smem, cudaStream_t st) {
    switch (epi) {
        case EPI_PLAIN: return launch_mt<OutT, EPI_PLAIN>(p, grid, smem, st);
        case EPI_RESID: return launch_mt<OutT, EPI_RESID>(p, grid, smem, st);
        case EPI_ACT: return launch_mt<OutT, EPI_ACT>(p, grid, smem, st);
        default: return -200;
    }
}

// The dequant epilogue alone, over int32 accumulators that already sit in global memory (summed across devices by a
// reduce-scatter of the partial products of a row-parallel linear).
template <typename OutT, int EPI>
__global__ void __launch_bounds__(256) epilogue_i32_kernel(const int32_t* __restrict__ acc, const float* __restrict__ xs,
                                                           const float* __restrict__ ws, const OutT* __restrict__ bias,
                                                           const OutT* __restrict__ rscale, const OutT* resid, OutT* D,
                                                           int64_t M, int64_t N, int act) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * N) return;
    const int64_t m = i / N, n = i - m * N;
    const float b = bias ? to_f<OutT>(bias[n]) : 0.f;
    const float rs = EPI == EPI_RESID ? to_f<OutT>(rscale[n]) : 0.f;
    const float rr = EPI == EPI_RESID ? to_f<OutT>(resid[i]) : 0.f;
    D[i] = from_f<OutT>(epilogue1<OutT, EPI>(acc[i], xs[m], ws[n], b, rs, rr, act));
}

template <typename OutT>
int launch_epilogue_i32(const int32_t* acc, const float* xs, const float* ws, const void* bias, const void* rscale,
                        const void* resid, void* D, int64_t M, int64_t N, int act, cudaStream_t st) {
    const unsigned grid = (unsigned)((M * N + 255) / 256);
    const OutT* b = (const OutT*)bias; const OutT* rs = (const OutT*)rscale; const OutT* rr = (const OutT*)resid;
    if (resid) epilogue_i32_kernel<OutT, EPI_RESID><<<grid, 256, 0, st>>>(acc, xs, ws, b, rs, rr, (OutT*)D, M, N, act);
    else if (act) epilogue_i32_kernel<OutT, EPI_ACT><<<grid, 256, 0, st>>>(acc, xs, ws, b, rs, rr, (OutT*)D, M, N, act);
    else epilogue_i32_kernel<OutT, EPI_PLAIN><<<grid, 256, 0, st>>>(acc, xs, ws, b, rs, rr, (OutT*)D, M, N, act);
    KCHECK();
    return 0;
}

}  // namespace

// New: D = epilogue(acc) for int32 accumulators [M, N] in global memory: the arithmetic of gpu_int8_gemm (resid == NULL,
// act == 0), gpu_int8_gemm_act (act != 0) or gpu_int8_gemm_residual (resid and rscale given). D may alias resid.
GPU_API int gpu_int8_epilogue(const int32_t* acc, const float* xs, const float* ws, const void* bias, const void* rscale,
                              const void* resid, void* D, int64_t M, int64_t N, int out_dt, int act, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if ((resid != nullptr) != (rscale != nullptr)) return -201;
    if (act < 0 || act > 3) return -204;
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dt == DT_F32) return launch_epilogue_i32<float>(acc, xs, ws, bias, rscale, resid, D, M, N, act, st);
    if (out_dt == DT_F16) return launch_epilogue_i32<half>(acc, xs, ws, bias, rscale, resid, D, M, N, act, st);
    if (out_dt == DT_BF16) return launch_epilogue_i32<bf16>(acc, xs, ws, bias, rscale, resid, D, M, N, act, st);
    return -200;
}

// ---- bias + residual over reduced partial outputs ------------------------------------------------------------------
// The tail of a row-parallel linear whose dequantized partial outputs were summed across devices (fast tensor-parallel
// mode): out[m, n0 + n] = T(T(y[m, n] + bias[n0 + n]) + resid[m, n0 + n]) for a column block [n0, n0 + Nc) of the
// output, y contiguous [M, Nc], resid and out with row pitch ld. 8 elements per thread, 16-byte accesses.
namespace {

template <typename T>
__global__ void __launch_bounds__(256) bias_residual_kernel(const T* __restrict__ y, const T* __restrict__ bias, const T* resid,
                                                            T* out, int64_t M, int Nc, int64_t ld, int n0) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= M * Nc) return;
    const int64_t m = i / Nc;
    const int n = (int)(i - m * Nc);
    float a[8], b[8], r[8];
    if constexpr (sizeof(T) == 2) {
        const uint4 ya = *reinterpret_cast<const uint4*>(y + i);
        const T* yh = reinterpret_cast<const T*>(&ya);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = to_f<T>(yh[e]);
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = to_f<T>(y[i + e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        b[e] = bias ? to_f<T>(bias[n0 + n + e]) : 0.f;
        r[e] = resid ? to_f<T>(resid[m * ld + n0 + n + e]) : 0.f;
    }
    T o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float v = bias ? rnd<T>(__fadd_rn(a[e], b[e])) : a[e];
        if (resid) v = __fadd_rn(v, r[e]);
        o[e] = from_f<T>(v);
    }
    T* dst = out + m * ld + n0 + n;
    if constexpr (sizeof(T) == 2) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
    else {
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[e] = o[e];
    }
}

}  // namespace

// New (tensor parallelism; the reference is single-device): out[:, n0:n0+Nc] = y + bias[n0:n0+Nc] + resid[:, n0:n0+Nc].
// y [M, Nc] contiguous in the activation dtype; bias [>= n0 + Nc] and resid [M, ld] nullable; out [M, ld] may alias resid.
// Nc, n0 and ld multiples of 8, pointers 16-byte aligned (-202).
GPU_API int gpu_bias_residual_add(const void* y, const void* bias, const void* resid, void* out, int64_t M, int64_t Nc,
                                  int64_t ld, int64_t n0, int dt, void* stream) {
    if (M <= 0 || Nc <= 0) return 0;
    if ((Nc | ld | n0) & 7 || (((uintptr_t)y | (uintptr_t)bias | (uintptr_t)resid | (uintptr_t)out) & 15)) return -202;
    if (Nc > INT32_MAX || n0 > INT32_MAX) return -200;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)((M * Nc / 8 + 255) / 256);
    if (dt == DT_F32) bias_residual_kernel<float><<<grid, 256, 0, st>>>((const float*)y, (const float*)bias, (const float*)resid, (float*)out, M, (int)Nc, ld, (int)n0);
    else if (dt == DT_F16) bias_residual_kernel<half><<<grid, 256, 0, st>>>((const half*)y, (const half*)bias, (const half*)resid, (half*)out, M, (int)Nc, ld, (int)n0);
    else if (dt == DT_BF16) bias_residual_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)y, (const bf16*)bias, (const bf16*)resid, (bf16*)out, M, (int)Nc, ld, (int)n0);
    else return -200;
    KCHECK();
    return 0;
}

// ---- K not a multiple of 16 ----------------------------------------------------------------------------------
// The tensor-core kernel stages its operands with TMA, which needs a 16-byte row pitch. The reference serves rows whose
// K is only a multiple of 8 with narrower-aligned tile configurations (csrc/vendor/cutlass_gemm_int8.cu:190-191,
// 265-267); such shapes (and 16-byte-misaligned operands) take this plain CUDA-core kernel here: 64 x 64 outputs per CTA,
// 64 bytes of K per step through shared memory, dp4a into int32 (exact), the same epilogue arithmetic. Rare shapes:
// built to be right, not fast.
namespace {

constexpr int kGT = 64;        // tile edge
constexpr int kGK = 64;        // bytes of K per step
constexpr int kGPitch = 17;    // words per staged row (16 + 1: conflict-free column reads)

template <typename OutT, int EPI>
__global__ void __launch_bounds__(256) generic_gemm_kernel(const SkinnyParams p, int vec) {
    __shared__ uint32_t a_s[kGT][kGPitch], w_s[kGT][kGPitch];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * kGT, n0 = blockIdx.x * kGT;
    int acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0;
    for (int k0 = 0; k0 < p.K; k0 += kGK) {
        // stage [64 rows][64 bytes] of A and of W, zero beyond M, N and K; `vec` bytes per load (8, 4 or 1)
        for (int idx = threadIdx.x; idx < 2 * kGT * (kGK / 8); idx += 256) {
            const bool is_w = idx >= kGT * (kGK / 8);
            const int j = is_w ? idx - kGT * (kGK / 8) : idx;
            const int r = j >> 3, c8 = j & 7;
            const int row = (is_w ? n0 : m0) + r, k = k0 + 8 * c8;
            const int8_t* src = (is_w ? p.W : p.A) + (int64_t)row * p.K + k;
            uint32_t lo = 0, hi = 0;
            if (row < (is_w ? p.N : p.M) && k < p.K) {
                if (vec == 8 && k + 8 <= p.K) {
                    const uint2 u = *reinterpret_cast<const uint2*>(src);
                    lo = u.x, hi = u.y;
                } else if (vec >= 4 && k + 8 <= p.K) {
                    lo = reinterpret_cast<const uint32_t*>(src)[0], hi = reinterpret_cast<const uint32_t*>(src)[1];
                } else {
                    for (int b = 0; b < 8 && k + b < p.K; ++b) {
                        const uint32_t v = (uint8_t)src[b];
                        if (b < 4) lo |= v << (8 * b); else hi |= v << (8 * (b - 4));
                    }
                }
            }
            uint32_t(*dst)[kGPitch] = is_w ? w_s : a_s;
            dst[r][2 * c8] = lo, dst[r][2 * c8 + 1] = hi;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kGK / 4; ++kk) {
            int a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = (int)a_s[ty + 16 * i][kk], w[i] = (int)w_s[tx + 16 * i][kk];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
            if (m >= p.M || n >= p.N) continue;
            const int64_t o = (int64_t)m * p.N + n;
            if (EPI == EPI_ACC) reinterpret_cast<int32_t*>(p.D)[o] = acc[i][j];
            else {
                const float bias = p.bias ? to_f<OutT>(reinterpret_cast<const OutT*>(p.bias)[n]) : 0.f;
                const float rs = EPI == EPI_RESID ? to_f<OutT>(reinterpret_cast<const OutT*>(p.rscale)[n]) : 0.f;
                const float rr = EPI == EPI_RESID ? to_f<OutT>(reinterpret_cast<const OutT*>(p.resid)[o]) : 0.f;
                reinterpret_cast<OutT*>(p.D)[o] = from_f<OutT>(epilogue1<OutT, EPI>(acc[i][j], p.xs[m], p.ws[n], bias, rs, rr, p.act));
            }
        }
}

template <typename OutT>
int launch_generic_epi(int epi, const SkinnyParams& p, dim3 grid, int vec, cudaStream_t st) {
    switch (epi) {
        case EPI_PLAIN: generic_gemm_kernel<OutT, EPI_PLAIN><<<grid, 256, 0, st>>>(p, vec); break;
        case EPI_RESID: generic_gemm_kernel<OutT, EPI_RESID><<<grid, 256, 0, st>>>(p, vec); break;
        case EPI_ACT: generic_gemm_kernel<OutT, EPI_ACT><<<grid, 256, 0, st>>>(p, vec); break;
        default: return -200;
    }
    KCHECK();
    return 0;
}

}  // namespace

int b200q::launch_generic_gemm(int epi, const SkinnyParams& p, int out_dt, cudaStream_t st) {
    const dim3 grid((unsigned)((p.N + kGT - 1) / kGT), (unsigned)((p.M + kGT - 1) / kGT));
    if (grid.y > 65535u) return -200;
    const uintptr_t al = (uintptr_t)p.A | (uintptr_t)p.W | (uintptr_t)p.K;
    const int vec = (al & 7) == 0 ? 8 : (al & 3) == 0 ? 4 : 1;
    if (epi == EPI_ACC) {
        generic_gemm_kernel<float, EPI_ACC><<<grid, 256, 0, st>>>(p, vec);
        KCHECK();
        return 0;
    }
    if (out_dt == DT_F32) return launch_generic_epi<float>(epi, p, grid, vec, st);
    if (out_dt == DT_F16) return launch_generic_epi<half>(epi, p, grid, vec, st);
    return launch_generic_epi<bf16>(epi, p, grid, vec, st);
}

bool b200q::skinny_gemm_applies(int64_t M, int64_t N, int64_t K) {
    return M >= 1 && M <= 8 && K % 16 == 0 && M * K <= 160 * 1024 && N >= 1;
}

int b200q::launch_skinny_gemm(int epi, const SkinnyParams& p, int out_dt, int sms, cudaStream_t st) {
    const size_t smem = (size_t)p.M * p.K;
    const int nblocks = (p.N + kRowsPerWarp - 1) / kRowsPerWarp;
    int grid = (nblocks + kWarps - 1) / kWarps;
    const int cap = sms * 4;
    if (grid > cap) grid = cap;
    if (epi == EPI_ACC) return launch_mt<float, EPI_ACC>(p, grid, smem, st);
    if (out_dt == DT_F32) return launch_epi<float>(epi, p, grid, smem, st);
    if (out_dt == DT_F16) return launch_epi<half>(epi, p, grid, smem, st);
    return launch_epi<bf16>(epi, p, grid, smem, st);
}
