// W6A8 GEMM: the CTA-pair kernel of gemm_i8.cu with the W operand arriving as 6-bit codes and expanded to int8 in
// shared memory. Included by gemm_i8.cu inside its anonymous namespace (shares its parameters and epilogue).
//
// Storage (the reference's, csrc/h3.cu:8-37, csrc/vendor/w6a8_requant.cu:128-151): a weight row is K/2 bytes of low
// nibbles (element e in byte e/2, even e in the low nibble) followed by K/4 bytes holding the top two bits of four
// consecutive elements; one fp8-e4m3 scale s_rel per G = 32 columns; the int8 the GEMM multiplies is
// clamp(rint((code - 32) * s_rel), +-127). The reference decodes the whole matrix to int8 before every GEMM
// (src/h3.rs:1208-1216); here the packed planes are what crosses HBM and L2 (0.78 bytes per weight).
//
// Per 128-byte K box and CTA: TMA brings bn/2 rows x 64 B of nibbles and x 32 B of top bits (64-byte and 32-byte
// swizzles, so that one thread per row reads without bank conflicts); eight unpack warps, two threads per weight
// row, expand them into the 128-byte-swizzled int8 tile the MMA descriptor expects, make the writes visible to the
// async proxy and arrive on the leader's "full" barrier, which also counts the A bytes. Four epilogue warps.
// The arithmetic is exact in half precision: code - 32 has 6 bits, e4m3 has 4, the product at most 10; rint is one
// addition of 1536 (ulp 1), ties to even, after the clamp.

constexpr int kW6EpiWarps = 4;
constexpr int kW6Groups = 3;                     // unpack groups of four warps, taking K boxes in turn
constexpr int kW6UnpackWarps = 4 * kW6Groups;
constexpr int kW6Threads = 32 * (2 + kW6EpiWarps + kW6UnpackWarps);
constexpr int kW6StagingPerWarp = 6144;   // output chunk (2 KB, or 4 KB for 4-byte outputs) + 3 KB of staged vectors
constexpr int kW6StagingBytes = kW6EpiWarps * kW6StagingPerWarp;

struct W6Extra {
    const uint8_t* s_rel;   // [N, K / 32] e4m3
    int srel_pitch;         // K / 32
    int sb;                 // depth of the ring of expanded tiles
};

// Whole-warp wait for the unpack warps: lane 0 polls (256 threads polling one shared-memory word would compete with
// the tensor core's operand reads), then every lane observes the completed phase itself, which is what orders its
// reads after the TMA writes.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait_suspended(bar, parity, abort_flag, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return false;
    return mbar_try_wait(bar, parity) || mbar_wait_suspended(bar, parity, abort_flag, code);
}

constexpr int kW6BStages = 4;    // ring of expanded W tiles: only has to span unpack -> MMA

// Rings: (A, packed planes) SA deep, filled by TMA far ahead of use; expanded W tiles kW6BStages deep, written by
// the unpack warps. Barriers: afull (leader: A bytes of both CTAs), pfull (per CTA: its packed planes), aempty (per
// CTA: MMAs have read A slot -> its packed slot is free too, the unpack that fed those MMAs being long done),
// bfull (leader: 16 unpack-warp arrivals), bempty (per CTA: MMAs have read the expanded slot).
// MH = 256-row halves per tile (1 or 2). With MH = 2 an expanded W tile feeds two sets of MMAs (rows 0-255 and 256-511 of
// the tile, two accumulators of bn <= 128 columns per buffer), so the unpack work per MMA halves.
template <typename OutT, int EPI, int MH>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kW6Threads, 1)
gemm_w6a8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_lo,
                      const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_d,
                      const GemmParams p, const W6Extra x6) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw_addr);
    const int SA = p.stages;
    const int SB = x6.sb;
    const int BN = p.bn;
    const int rows_w = BN / 2;                              // weight rows this CTA expands
    constexpr uint32_t a_box = BM * BK;                    // one 128-row, 128-byte K box of A
    const uint32_t a_bytes = MH * a_box, b_bytes = (uint32_t)rows_w * BK, lo_bytes = (uint32_t)rows_w * 64, hi_bytes = (uint32_t)rows_w * 32;
    uint8_t* staging = sm;
    const uint32_t sA = base + kW6StagingBytes;
    const uint32_t sB = sA + SA * a_bytes;
    const uint32_t sLo = sB + SB * b_bytes;
    const uint32_t sHi = sLo + SA * lo_bytes;
    uint8_t* tail = sm + kW6StagingBytes + SA * (a_bytes + lo_bytes + hi_bytes) + SB * b_bytes;
    const uint32_t bar_afull = smem_u32(tail);
    const uint32_t bar_aempty = bar_afull + 8 * kMaxStages;
    const uint32_t bar_pfull = bar_aempty + 8 * kMaxStages;
    const uint32_t bar_bfull = bar_pfull + 8 * kMaxStages;
    const uint32_t bar_bempty = bar_bfull + 8 * kMaxStages;
    const uint32_t bar_tfull = bar_bempty + 8 * kMaxStages;
    const uint32_t bar_tempty = bar_tfull + 16;
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(tail + 8 * (5 * kMaxStages + 4));
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_ptr_s + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int nclusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < SA; ++i) {
            mbar_init(bar_afull + 8 * i, 1);
            mbar_init(bar_aempty + 8 * i, 1);
            mbar_init(bar_pfull + 8 * i, 1);
        }
        for (int i = 0; i < SB; ++i) {
            mbar_init(bar_bfull + 8 * i, 2 * 4);   // the four warps of one group in each CTA
            mbar_init(bar_bempty + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 2 * kW6EpiWarps);
        }
        *abort_s = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a), prefetch_tmap(&tmap_lo), prefetch_tmap(&tmap_hi);
        if (p.tma_store) prefetch_tmap(&tmap_d);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_ptr_s), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    if (warp == 0) {
        // ---------------- TMA producer: A tile (credited to the leader) and this CTA's packed planes ----------------
        if (lane == 0) {
            int sa = 0;
            uint32_t pa = 0;
            bool ok = true;
            for (int t = cluster_id; t < p.num_tiles && ok; t += nclusters) {
                int tm, tn;
                tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
                const int row_a = tm * (2 * BM * MH) + (int)rank * BM;
                const int row_w = tn * BN + (int)rank * rows_w;
                for (int kb = 0; kb < p.k_iters; ++kb) {
                    if (!mbar_wait_suspended(bar_aempty + 8 * sa, pa ^ 1u, abort_s, ST_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_arrive_expect_tx(bar_pfull + 8 * sa, lo_bytes + hi_bytes);
                    tma_load_2d(sLo + sa * lo_bytes, &tmap_lo, kb * 64, row_w, bar_pfull + 8 * sa);
                    tma_load_2d(sHi + sa * hi_bytes, &tmap_hi, kb * 32, row_w, bar_pfull + 8 * sa);
                    if (leader) mbar_arrive_expect_tx(bar_afull + 8 * sa, 2 * a_bytes);
#pragma unroll
                    for (int h = 0; h < MH; ++h)
                        tma_load_2d_pair(sA + sa * a_bytes + h * a_box, &tmap_a, kb * BK, row_a + h * 2 * BM,
                                         mapa_shared(bar_afull + 8 * sa, 0));
                    if (++sa == SA) { sa = 0; pa ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA) ----------------
        if (leader && lane == 0) {
            const uint32_t a_lo0 = umma_desc_lo(sA), b_lo0 = umma_desc_lo(sB);
            const uint32_t a_step = a_bytes >> 4, b_step = b_bytes >> 4;
            const uint32_t idesc = p.idesc;
            int sa = 0, sb = 0;
            uint32_t pa = 0, pb = 0;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            int buf = 0;
            uint32_t tphase = 0;
            bool ok = true;
            for (int t = cluster_id; t < p.num_tiles && ok; t += nclusters) {
                {
                    if (!mbar_wait(bar_tempty + 8 * buf, tphase ^ 1u, abort_s, ST_TIMEOUT_TMEM_EMPTY)) break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256;
                for (int kb = 0; kb < p.k_iters; ++kb) {
                    if (!mbar_wait(bar_afull + 8 * sa, pa, abort_s, ST_TIMEOUT_FULL)) { ok = false; break; }
                    if (!mbar_wait(bar_bfull + 8 * sb, pb, abort_s, ST_TIMEOUT_FULL)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int h = 0; h < MH; ++h) {
                        const uint32_t dh = d_tmem + h * 128, ah = a_lo + h * (a_box >> 4);
                        umma_pair_lo<0>(dh, ah, b_lo, idesc, kb);
                        umma_pair_lo<0>(dh, ah + 2, b_lo + 2, idesc, 1);
                        umma_pair_lo<0>(dh, ah + 4, b_lo + 4, idesc, 1);
                        umma_pair_lo<0>(dh, ah + 6, b_lo + 6, idesc, 1);
                    }
                    umma_commit_pair(bar_bempty + 8 * sb);
                    umma_commit_pair(bar_aempty + 8 * sa);
                    ++sa, a_lo += a_step;
                    if (sa == SA) sa = 0, pa ^= 1u, a_lo = a_lo0;
                    ++sb, b_lo += b_step;
                    if (sb == SB) sb = 0, pb ^= 1u, b_lo = b_lo0;
                }
                if (!ok) break;
                umma_commit_pair(bar_tfull + 8 * buf);
                buf ^= 1;
                if (buf == 0) tphase ^= 1u;
            }
        }
    } else if (warp >= 2 + kW6EpiWarps) {
        // ---------------- unpack warps: groups of four warps take K boxes in turn; one thread per weight row ----------------
        // Every barrier operation and the proxy fence cost a warp on the order of a hundred cycles whatever the amount of
        // data, so a group pays them once per 128 elements of its rows, and the groups overlap one another's waits.
        const int uw = warp - (2 + kW6EpiWarps);
        const int grp = uw >> 2;
        // up to 64 rows per CTA (bn <= 128): two threads per row, 64 elements each; else one thread per row
        const bool two = rows_w <= 64;
        const int r = two ? 32 * (uw & 1) + lane : 32 * (uw & 3) + lane;      // row of the half tile
        const int hf = two ? (uw >> 1) & 1 : 0;                               // which 64 elements of the box
        const bool has_row = r < rows_w;
        const uint32_t bfull_leader = mapa_shared(bar_bfull, 0);
        const int sw_lo = (r >> 1) & 3, sw_hi = (r >> 2) & 1, sw_out = r & 7;
        const bool wide = (x6.srel_pitch & 15) == 0 && ((uintptr_t)x6.s_rel & 15) == 0;   // scale rows readable 16 bytes at a time
        int sa = 0, sb = 0, turn = 0;           // turn: which group takes the current K box
        uint32_t pa = 0, pb = 0;
        bool ok = true;
        for (int t = cluster_id; t < p.num_tiles && ok; t += nclusters) {
            int tm, tn;
            tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
            const int n = min(tn * BN + (int)rank * rows_w + r, p.N - 1);
            const uint8_t* srow = x6.s_rel + (size_t)n * x6.srel_pitch;
            // scale bytes of four K boxes at a time, fetched four boxes ahead of their use
            uint4 sc_cur = make_uint4(0, 0, 0, 0), sc_next = make_uint4(0, 0, 0, 0);
            auto fetch = [&](int kb4) -> uint4 {     // scales of boxes 4*kb4 .. 4*kb4+3
                uint4 v = make_uint4(0x38383838u, 0x38383838u, 0x38383838u, 0x38383838u);
                if (!has_row) return v;
                if (wide && 4 * kb4 + 4 <= p.k_iters) return __ldg(reinterpret_cast<const uint4*>(srow) + kb4);
                const uint32_t* s32 = reinterpret_cast<const uint32_t*>(srow) + 4 * kb4;
                const int left = p.k_iters - 4 * kb4;
                if (left > 0) v.x = __ldg(s32);
                if (left > 1) v.y = __ldg(s32 + 1);
                if (left > 2) v.z = __ldg(s32 + 2);
                if (left > 3) v.w = __ldg(s32 + 3);
                return v;
            };
            sc_next = fetch(0);
            for (int kb = 0; kb < p.k_iters; ++kb) {
                if ((kb & 3) == 0) {
                    sc_cur = sc_next;
                    if (kb + 4 < p.k_iters) sc_next = fetch((kb >> 2) + 1);
                }
                if (turn == grp) {
                    const int q = kb & 3;
                    const uint32_t sr = q == 0 ? sc_cur.x : q == 1 ? sc_cur.y : q == 2 ? sc_cur.z : sc_cur.w;
                    // usually both are complete already: one probe by every lane, the polling form only when not
                    if (!__all_sync(0xffffffffu, mbar_try_wait(bar_pfull + 8 * sa, pa)) &&
                        !mbar_wait_warp(bar_pfull + 8 * sa, pa, abort_s, ST_TIMEOUT_UNPACK)) { ok = false; break; }
                    if (!__all_sync(0xffffffffu, mbar_try_wait(bar_bempty + 8 * sb, pb ^ 1u)) &&
                        !mbar_wait_warp(bar_bempty + 8 * sb, pb ^ 1u, abort_s, ST_TIMEOUT_UNPACK)) { ok = false; break; }
                    {
                        const int rr = has_row ? r : 0;    // lanes beyond the tile's rows redo row 0 (warp votes below) and store nothing
                        const uint8_t* lo = sm + (sLo - base) + sa * lo_bytes + rr * 64;
                        const uint8_t* hi = sm + (sHi - base) + sa * hi_bytes + rr * 32;
                        uint8_t* out = sm + (sB - base) + sb * b_bytes + rr * 128;
                        const uint4 h0 = *reinterpret_cast<const uint4*>(hi + ((hf ^ sw_hi) << 4));
                        const uint4 h1 = *reinterpret_cast<const uint4*>(hi + ((1 ^ sw_hi) << 4));
                        const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                        for (int c = 0; c < 4; ++c) {      // 32 elements = one scale group per 16-byte piece of nibbles
                            if (two && (c >> 1) != hf) continue;             // the other thread of the row (the same for the whole warp)
                            const int hi_w = two ? 2 * (c & 1) : 2 * c;
                            const uint4 l = *reinterpret_cast<const uint4*>(lo + ((c ^ sw_lo) << 4));
                            uint32_t o[8];
                            w6_group(l, hw[hi_w], hw[hi_w + 1], (sr >> (8 * c)) & 0xffu, o);
                            if (has_row) {
                                *reinterpret_cast<uint4*>(out + (((2 * c) ^ sw_out) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                                *reinterpret_cast<uint4*>(out + (((2 * c + 1) ^ sw_out) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                            }
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(bfull_leader + 8 * sb);
                }
                if (++turn == kW6Groups) turn = 0;
                if (++sa == SA) { sa = 0; pa ^= 1u; }
                if (++sb == SB) { sb = 0; pb ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue: four warps, each draining every 32-column chunk of its TMEM lane quarter ----------------
        constexpr int kEsz = EPI == EPI_ACC ? 4 : (int)sizeof(OutT);
        constexpr bool kStageVec = kEsz == 2;            // 2-byte outputs: 2 KB chunk + 3 KB of per-column vectors
        const int ew = warp - 2;
        const int quad = warp & 3;
        const int nchunks = BN / 32;
        uint8_t* my_stage = staging + ew * kW6StagingPerWarp;
        const uint32_t my_stage_u32 = smem_u32(my_stage);
        float* my_vec = reinterpret_cast<float*>(my_stage + 2048);   // ws[256] | bias[256] | rscale[256]
        int buf = 0;
        uint32_t tphase = 0;
        for (int t = cluster_id; t < p.num_tiles; t += nclusters) {
            int tm, tn;
            tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
            const int n0 = tn * BN;
            const bool staged = kStageVec && p.tma_store;
            if (staged) {
                // the tile's columns of ws / bias / rscale, fetched while the mainloop still runs
                if (lane == 0) bulk_wait_read<0>();
                __syncwarp();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int n = n0 + 32 * k + lane;
                    const bool in = n < p.N && k < nchunks;
                    my_vec[32 * k + lane] = in ? p.ws[n] : 0.f;
                    my_vec[256 + 32 * k + lane] = (in && p.bias) ? to_f<OutT>(reinterpret_cast<const OutT*>(p.bias)[n]) : 0.f;
                    if (EPI == EPI_RESID)
                        my_vec[512 + 32 * k + lane] = in ? to_f<OutT>(reinterpret_cast<const OutT*>(p.rscale)[n]) : 0.f;
                }
                __syncwarp();
            }
            if (!mbar_wait_warp_relaxed(bar_tfull + 8 * buf, tphase, abort_s, ST_TIMEOUT_TMEM_FULL)) break;
            tc_fence_after();
            uint32_t ra[32];
#pragma unroll 1
            for (int hc = 0; hc < MH * nchunks; ++hc) {
                const int h = MH == 1 ? 0 : hc / nchunks, c = hc - h * nchunks;
                const int row0 = tm * (2 * BM * MH) + h * 2 * BM + (int)rank * BM + quad * 32;
                const int row = row0 + lane;
                const bool row_ok = row < p.M;
                const int rrow = row_ok ? row : p.M - 1;
                const float xs_r = EPI != EPI_ACC ? p.xs[rrow] : 0.f;
                const uint32_t taddr = tmem_base + buf * 256 + h * 128 + ((uint32_t)(quad * 32) << 16);
                tmem_ld32(taddr + c * 32, ra);
                tmem_ld_wait();
                const int col0 = n0 + c * 32;
                if (col0 >= p.N) continue;
                if (p.tma_store) {
                    if constexpr (kStageVec) {
                        uint4 pk[4];
                        chunk_compute16<OutT, EPI, 256>(p, ra, rrow, col0, xs_r, my_vec + 32 * c, pk);
                        if (lane == 0) bulk_wait_read<0>();   // the previous chunk's store has read the buffer
                        __syncwarp();
                        chunk_write16(pk, my_stage, lane);
                    } else {
                        if (lane == 0) bulk_wait_read<0>();
                        __syncwarp();
                        chunk_to_smem<OutT, EPI>(p, ra, rrow, col0, xs_r, my_stage, lane);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmap_d, my_stage_u32, col0, row0);
                        bulk_commit();
                    }
                } else if (row_ok) {
                    chunk_direct<OutT, EPI>(p, ra, row, col0, xs_r);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * buf, 0));
            buf ^= 1;
            if (buf == 0) tphase ^= 1u;
        }
        if (p.tma_store && lane == 0) bulk_wait_read<0>();   // the staged rows have been read; the grid's end completes the writes
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (*abort_s != 0) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicCAS(&g_kernel_status, 0, *abort_s);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
// Tensor map of one plane of the packed rows: `cols` bytes per row at `pitch` bytes, boxes of box_x bytes x box_rows.
bool make_plane_tmap(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols, int64_t pitch, int box_x, int box_rows,
                     CUtensorMapSwizzle swz) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch};
    const cuuint32_t box[2] = {(cuuint32_t)box_x, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename OutT, int EPI, int MH>
int launch_w6_mh(const CUtensorMap& ta, const CUtensorMap& tlo, const CUtensorMap& thi, const CUtensorMap& td,
                 const GemmParams& p, const W6Extra& x6, int grid, cudaStream_t st) {
    auto kern = gemm_w6a8_pair_kernel<OutT, EPI, MH>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured.fetch_or(bit, std::memory_order_release);
    }
    kern<<<grid, kW6Threads, kSmemBytes, st>>>(ta, tlo, thi, td, p, x6);
    KCHECK();
    return 0;
}

template <typename OutT, int EPI>
int launch_w6(const CUtensorMap& ta, const CUtensorMap& tlo, const CUtensorMap& thi, const CUtensorMap& td,
              const GemmParams& p, const W6Extra& x6, int mh, int grid, cudaStream_t st) {
    return mh == 2 ? launch_w6_mh<OutT, EPI, 2>(ta, tlo, thi, td, p, x6, grid, st)
                   : launch_w6_mh<OutT, EPI, 1>(ta, tlo, thi, td, p, x6, grid, st);
}

int run_w6_gemm(int epi, const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, const float* xs, const float* ws,
                const void* bias, const void* rscale, const void* resid, void* D, int64_t M, int64_t N, int64_t K, int G,
                int out_dt, cudaStream_t st, int act = 0) {
    if (M == 0 || N == 0) return 0;
    if (G != 32) return -206;                                  // the fused unpack is built for the reference's group size
    if (epi == EPI_RESID && (!rscale || !resid)) return -201;
    if (epi != EPI_ACC && (out_dt < 0 || out_dt > 2)) return -200;
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return -200;
    // whole 128-element K boxes; planes and scale rows must be addressable by TMA / 32-bit loads
    if (K <= 0 || (K % 128) != 0 || ((uintptr_t)A & 15) || ((uintptr_t)Wq6 & 15) || ((uintptr_t)s_rel & 3)) return -202;
    int dev = 0;
    cudaGetDevice(&dev);
    const int clusters = device_sm_count(dev) / 2;
    GemmParams p{};
    p.xs = xs, p.ws = ws, p.bias = bias, p.rscale = rscale, p.resid = resid, p.D = D;
    p.M = (int)M, p.N = (int)N, p.K = (int)K;
    p.act = act;
    p.act_lut = nullptr;
    const int esz = epi == EPI_ACC ? 4 : (out_dt == DT_F32 ? 4 : 2);
    auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    p.vec_ok = (N % 8 == 0) && al16(D) && al16(ws) && al16(bias) && al16(rscale) && al16(resid);
    p.tma_store = al16(D) && ((N * esz) % 16 == 0);
    p.ksub = 1;
    p.k_iters = (int)(K / BK);
    // More than 256 rows: tiles of 512 rows x 128 columns, so that each expanded W tile serves two sets of MMAs and the
    // unpack work per MMA halves; otherwise one 256-row half and the column width that fills the clusters best.
    const int mh = M > 256 && N >= 128 ? 2 : 1;
    const int bn = mh == 2 ? 128 : choose_bn(M, N, clusters);
    p.bn = bn;
    p.idesc = umma_idesc_i8(2 * BM, bn);
    const int stage_bytes = mh * BM * BK + (bn / 2) * (64 + 32);     // A boxes + packed planes; the expanded ring is separate
    const int sbs = kW6BStages;
    const int stages = (kSmemBytes - 1024 - 512 - kW6StagingBytes - sbs * (bn / 2) * BK) / stage_bytes;
    p.stages = stages > kMaxStages ? kMaxStages : stages;
    p.tiles_m = (int)((M + 2 * BM * mh - 1) / (2 * BM * mh));
    p.tiles_n = (int)((N + bn - 1) / bn);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.whole_tiles = p.num_tiles, p.num_items = p.num_tiles, p.kps = p.k_iters;
    const int64_t pitch = 3 * K / 4;
    CUtensorMap ta, tlo, thi, td;
    if (!make_operand_tmap(&ta, A, M, K, BM)) return -203;
    if (!make_plane_tmap(&tlo, Wq6, N, K / 2, pitch, 64, bn / 2, CU_TENSOR_MAP_SWIZZLE_64B)) return -203;
    if (!make_plane_tmap(&thi, Wq6 + K / 2, N, K / 4, pitch, 32, bn / 2, CU_TENSOR_MAP_SWIZZLE_32B)) return -203;
    if (p.tma_store) {
        if (!make_output_tmap(&td, D, M, N, esz)) return -203;
    } else {
        td = ta;
    }
    W6Extra x6{s_rel, (int)(K / 32), sbs};
    const int grid = 2 * (p.num_tiles < clusters ? p.num_tiles : clusters);
    if (epi == EPI_ACC) return launch_w6<float, EPI_ACC>(ta, tlo, thi, td, p, x6, mh, grid, st);
#define W6_DISPATCH(T)                                                                                   \
    (epi == EPI_RESID ? launch_w6<T, EPI_RESID>(ta, tlo, thi, td, p, x6, mh, grid, st)                      \
     : epi == EPI_ACT ? launch_w6<T, EPI_ACT>(ta, tlo, thi, td, p, x6, mh, grid, st)                        \
                      : launch_w6<T, EPI_PLAIN>(ta, tlo, thi, td, p, x6, mh, grid, st))
    if (out_dt == DT_F32) return W6_DISPATCH(float);
    if (out_dt == DT_F16) return W6_DISPATCH(half);
    return W6_DISPATCH(bf16);
#undef W6_DISPATCH
}
