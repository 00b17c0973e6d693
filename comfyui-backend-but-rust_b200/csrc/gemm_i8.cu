// int8 x int8 -> int32 GEMM with the fused dequant epilogue, for sm_100a.
//
//   D[m,n] = out( (sum_k A[m,k] * W[n,k]) * xs[m] * ws[n] + bias[n] )                       gpu_int8_gemm
//   D[m,n] = out( resid[m,n] + rscale[n] * out( acc * xs[m] * ws[n] + bias[n] ) )            gpu_int8_gemm_residual
//   D[m,n] = out( act( out( acc * xs[m] * ws[n] + bias[n] ) ) )                              gpu_int8_gemm_act (new)
//
// These are the entry points the reference exports from csrc/gemm.cu:123-140 over its CUTLASS 2.x
// mma.sync kernels (csrc/vendor/cutlass_gemm_int8.cu); the rounding points are those of its epilogue
// visitor trees (:84-95 plain, :143-161 residual).
//
// One persistent CTA per SM, 192 threads:
//   warp 0      TMA producer: 128-byte-swizzled int8 tiles of A [128 x 128] and W [BN x 128] into a ring of
//               shared-memory stages (cp.async.bulk.tensor, no multicast), completion on mbarriers
//   warp 1      allocates tensor memory; one thread issues tcgen05.mma kind::i8 (M=128, N=BN, K=32), four per
//               stage, and commits each stage back to the producer and each finished tile to the epilogue
//   warps 2-5   epilogue: tcgen05.ld the int32 accumulator (two TMEM buffers, so the epilogue of tile i runs
//               under the mainloop of tile i+1), scale, bias, optional activation or residual, round, store
// Every wait is bounded; a wait that runs out records a code in g_kernel_status and the CTA unwinds.
#include <atomic>
#include <cuda.h>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

__device__ int g_kernel_status = 0;

namespace {

constexpr int BM = 128;        // rows of A per tile = UMMA M = TMEM lanes
constexpr int BK = 128;        // int8 elements (= bytes) of K per stage: one 128-byte swizzle row
constexpr int UMMA_K = 32;     // K of one tcgen05.mma kind::i8
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;

enum EpiMode { EPI_PLAIN = 0, EPI_RESID = 1, EPI_ACT = 2, EPI_ACC = 3 };
enum Act { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_GELU_ERF = 3 };

struct GemmParams {
    const float* xs;     // [M]
    const float* ws;     // [N]
    const void* bias;    // [N] out dtype, nullable
    const void* rscale;  // [N] out dtype (residual form)
    const void* resid;   // [M,N] out dtype (residual form), may alias D
    void* D;             // [M,N] out dtype, or int32 for EPI_ACC
    int M, N, K;
    int tiles_m, tiles_n, num_tiles, k_iters;
    int act;
    int contract;        // bit 0: acc*xs*ws + bias ends in one fma; bit 1: y*rscale + resid is one fma
    int vec_ok;          // rows of D (and resid) start 16-byte aligned and N % 8 == 0
};

template <int BN> struct Cfg {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers; 512 or 256 columns
    // tiles | barriers + tmem pointer + abort flag | 1024 B alignment slack
    static constexpr int kSmemBytes = kStages * kStageBytes + 256 + 1024;
};

// Tile order: bands of 8 row tiles, column tile fastest-varying across the band's rows, so that the CTAs
// running at one time share a few A row-panels and W column-panels in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    constexpr int GROUP_M = 8;
    const int per_group = GROUP_M * tiles_n;
    const int group = t / per_group;
    const int first_m = group * GROUP_M;
    const int gsize = min(GROUP_M, tiles_m - first_m);
    const int r = t - group * per_group;
    tm = first_m + r % gsize;
    tn = r / gsize;
}

template <typename OutT> __device__ __forceinline__ void store8(OutT* p, const float (&y)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&y)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(y[0], y[1], y[2], y[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(y[4], y[5], y[6], y[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* p, const float (&y)[8]) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
}
template <> __device__ __forceinline__ void store8<half>(half* p, const float (&y)[8]) {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
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

template <int BN, typename OutT, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const GemmParams p) {
    using C = Cfg<BN>;
    constexpr int S = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled operand tiles need a 1024-byte aligned base
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw_addr);
    const uint32_t sA = base;                          // S x [128 x 128]
    const uint32_t sB = base + S * C::kABytes;         // S x [BN x 128]
    uint8_t* tail = sm + S * C::kStageBytes;
    const uint32_t bar_full = smem_u32(tail);             // S barriers
    const uint32_t bar_empty = bar_full + 8 * S;          // S
    const uint32_t bar_tfull = bar_empty + 8 * S;         // 2
    const uint32_t bar_tempty = bar_tfull + 16;           // 2
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(tail + 8 * (2 * S + 4));
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_ptr_s + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, kEpiThreads);
        }
        *abort_s = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_ptr_s), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
                for (int kb = 0; kb < p.k_iters; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_s, ST_TIMEOUT_EMPTY)) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_arrive_expect_tx(full, C::kStageBytes);
                    tma_load_2d(sA + stage * C::kABytes, &tmap_a, kb * BK, tm * BM, full);
                    tma_load_2d(sB + stage * C::kBBytes, &tmap_w, kb * BK, tn * BN, full);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t tphase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
                if (!mbar_wait(bar_tempty + 8 * buf, tphase ^ 1u, abort_s, ST_TIMEOUT_TMEM_EMPTY)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < p.k_iters; ++kb) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_s, ST_TIMEOUT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(sA + stage * C::kABytes);
                    const uint64_t db = umma_desc_sw128(sB + stage * C::kBBytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advancing the start address by 32 bytes inside the swizzle row selects the next K slice
                        umma_i8(d_tmem, da + (uint64_t)(k * UMMA_K / 16), db + (uint64_t)(k * UMMA_K / 16), idesc,
                                (kb | k) != 0);
                    }
                    umma_commit(bar_empty + 8 * stage);  // stage is free once these MMAs have read it
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(bar_tfull + 8 * buf);  // accumulator complete
                buf ^= 1;
                if (buf == 0) tphase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quad = warp & 3;         // the TMEM lane quarter this warp may read
        int buf = 0;
        uint32_t tphase = 0;
        for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
            int tm, tn;
            tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
            const int n0 = tn * BN;
            // the whole warp takes the same way out, so that the aligned TMEM loads below stay warp-wide
            const bool got = mbar_wait(bar_tfull + 8 * buf, tphase, abort_s, ST_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after();
            const int row = tm * BM + quad * 32 + lane;
            const bool row_ok = row < p.M;
            const float xs_r = (EPI != EPI_ACC && row_ok) ? p.xs[row] : 0.f;
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                tmem_ld_wait();
                if (!row_ok) continue;
                const int col0 = n0 + c * 32;
                if (EPI == EPI_ACC) {
                    int32_t* d = reinterpret_cast<int32_t*>(p.D) + (int64_t)row * p.N + col0;
                    if (p.vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<uint4*>(d + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.N) d[j] = (int32_t)r[j];
                    }
                    continue;
                }
                OutT* d = reinterpret_cast<OutT*>(p.D) + (int64_t)row * p.N + col0;
                const OutT* rsd = reinterpret_cast<const OutT*>(p.resid) + (int64_t)row * p.N + col0;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    if (col0 + j >= p.N) break;
                    const bool vec = p.vec_ok && col0 + j + 8 <= p.N;
                    // per-column vectors: every lane reads the same addresses (one broadcast per load)
                    float w8[8], b8[8], rs8[8], rr[8];
                    if (vec) {
                        load8<float>(p.ws + col0 + j, w8);
                        if (p.bias) load8<OutT>(reinterpret_cast<const OutT*>(p.bias) + col0 + j, b8);
                        if (EPI == EPI_RESID) {
                            load8<OutT>(reinterpret_cast<const OutT*>(p.rscale) + col0 + j, rs8);
                            load8<OutT>(rsd + j, rr);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int n = col0 + j + e;
                            const bool in = n < p.N;
                            w8[e] = in ? p.ws[n] : 0.f;
                            if (p.bias) b8[e] = in ? to_f<OutT>(reinterpret_cast<const OutT*>(p.bias)[n]) : 0.f;
                            if (EPI == EPI_RESID) {
                                rs8[e] = in ? to_f<OutT>(reinterpret_cast<const OutT*>(p.rscale)[n]) : 0.f;
                                rr[e] = in ? to_f<OutT>(rsd[j + e]) : 0.f;
                            }
                        }
                    }
                    if (!p.bias) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) b8[e] = 0.f;
                    }
                    float y[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float t0 = __fmul_rn(__int2float_rn((int)r[j + e]), xs_r);
                        float v = (p.contract & 1) ? __fmaf_rn(t0, w8[e], b8[e]) : __fadd_rn(__fmul_rn(t0, w8[e]), b8[e]);
                        v = rnd<OutT>(v);
                        if (EPI == EPI_RESID) {
                            v = (p.contract & 2) ? __fmaf_rn(v, rs8[e], rr[e]) : __fadd_rn(__fmul_rn(v, rs8[e]), rr[e]);
                        } else if (EPI == EPI_ACT) {
                            v = p.act == ACT_GELU_TANH ? gelu_tanh_f(v) : p.act == ACT_SILU ? silu_f(v) : gelu_f(v);
                        }
                        y[e] = v;
                    }
                    if (vec) store8<OutT>(d + j, y);
                    else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (col0 + j + e < p.N) d[j + e] = from_f<OutT>(y[e]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty + 8 * buf);
            buf ^= 1;
            if (buf == 0) tphase ^= 1u;
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_s != 0) {
        // a wait ran out: leave time for copies and MMAs still in flight, then report
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicCAS(&g_kernel_status, 0, *abort_s);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
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

// Tensor map of a row-major int8 matrix [rows, cols] (cols contiguous), box 128 bytes x box_rows, 128-byte swizzle.
// Rows and columns beyond the matrix read as zero.
bool make_tmap(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
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

struct DeviceInfo {
    int sm_count = 0;
};
DeviceInfo& device_info(int dev) {
    static DeviceInfo info[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    DeviceInfo& d = info[dev & 63];
    if (d.sm_count == 0) cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    return d;
}

std::atomic<int> g_contract{0};

template <int BN, typename OutT, int EPI>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tw, const GemmParams& p, int grid, cudaStream_t st) {
    auto kern = gemm_i8_kernel<BN, OutT, EPI>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured.fetch_or(bit, std::memory_order_release);
    }
    kern<<<grid, kThreads, Cfg<BN>::kSmemBytes, st>>>(ta, tw, p);
    KCHECK();
    return 0;
}

template <int BN, typename OutT>
int launch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tw, const GemmParams& p, int grid, cudaStream_t st) {
    switch (epi) {
        case EPI_PLAIN: return launch_gemm<BN, OutT, EPI_PLAIN>(ta, tw, p, grid, st);
        case EPI_RESID: return launch_gemm<BN, OutT, EPI_RESID>(ta, tw, p, grid, st);
        case EPI_ACT: return launch_gemm<BN, OutT, EPI_ACT>(ta, tw, p, grid, st);
        default: return -200;
    }
}

// Chooses the column-tile width: 256 unless 128 loses fewer SM-slots to the last partial wave.
int choose_bn(int64_t M, int64_t N, int sms) {
    const int64_t tm = (M + BM - 1) / BM;
    auto cost = [&](int bn, double per_tile) {
        const double tiles = (double)(tm * ((N + bn - 1) / bn));
        const double waves = tiles / sms;
        return ceil(waves) * per_tile;  // time in units of one 128x256 tile
    };
    return cost(256, 1.0) <= cost(128, 0.54) ? 256 : 128;
}

int run_gemm(int epi, const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias,
             const void* rscale, const void* resid, void* D, int64_t M, int64_t N, int64_t K, int out_dt, int act,
             cudaStream_t st) {
    if (M == 0 || N == 0) return 0;
    if (K == 0) return epi == EPI_RESID ? -201 : 0;  // the reference declines K == 0 for the residual form only
    if (epi == EPI_RESID && (!rscale || !resid)) return -201;
    if (epi != EPI_ACC && (out_dt < 0 || out_dt > 2)) return epi == EPI_RESID ? -201 : -200;
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return -200;
    // TMA needs 16-byte aligned bases and row pitch
    if ((K % 16) != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return -202;
    int dev = 0;
    cudaGetDevice(&dev);
    const int sms = device_info(dev).sm_count;
    const int bn = choose_bn(M, N, sms);
    CUtensorMap ta, tw;
    if (!make_tmap(&ta, A, M, K, BM) || !make_tmap(&tw, W, N, K, bn)) return -203;
    GemmParams p{};
    p.xs = xs, p.ws = ws, p.bias = bias, p.rscale = rscale, p.resid = resid, p.D = D;
    p.M = (int)M, p.N = (int)N, p.K = (int)K;
    p.tiles_m = (int)((M + BM - 1) / BM);
    p.tiles_n = (int)((N + bn - 1) / bn);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.k_iters = (int)((K + BK - 1) / BK);
    p.act = act;
    p.contract = g_contract.load(std::memory_order_relaxed);
    const int esz = epi == EPI_ACC ? 4 : (out_dt == DT_F32 ? 4 : 2);
    const int per16 = 16 / esz;
    auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    p.vec_ok = (N % 8 == 0) && (N % per16 == 0) && al16(D) && al16(ws) && al16(bias) && al16(rscale) && al16(resid);
    const int grid = p.num_tiles < sms ? p.num_tiles : sms;
#define BN_DISPATCH(BN_)                                                                          \
    if (epi == EPI_ACC) return launch_gemm<BN_, float, EPI_ACC>(ta, tw, p, grid, st);             \
    if (out_dt == DT_F32) return launch_epi<BN_, float>(epi, ta, tw, p, grid, st);                \
    if (out_dt == DT_F16) return launch_epi<BN_, half>(epi, ta, tw, p, grid, st);                 \
    return launch_epi<BN_, bf16>(epi, ta, tw, p, grid, st);
    if (bn == 256) { BN_DISPATCH(256) }
    BN_DISPATCH(128)
#undef BN_DISPATCH
}

}  // namespace

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

// New, for tests: the raw int32 accumulators D[m,n] = sum_k A[m,k]*W[n,k], which the fused forms never expose.
GPU_API int gpu_int8_gemm_acc_i32(const int8_t* A, const int8_t* W, int32_t* D, int64_t M, int64_t N, int64_t K,
                                  void* stream) {
    return run_gemm(EPI_ACC, A, W, nullptr, nullptr, nullptr, nullptr, nullptr, D, M, N, K, 0, 0, (cudaStream_t)stream);
}

// Which float forms the epilogue uses: bit 0 fuses (acc*xs)*ws + bias into one fma, bit 1 fuses y*rscale + resid.
// The default matches the reference binary's epilogue as compiled by nvcc 12.9 for sm_100a.
GPU_API void gpu_kernels_set_epilogue_contract(int bits) { g_contract.store(bits & 3); }

// Reads and clears the device status word (synchronises the device). 0 = no kernel gave up a wait.
GPU_API int gpu_kernels_status(int* status) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_kernel_status, &zero, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (status) *status = v;
    return 0;
}
