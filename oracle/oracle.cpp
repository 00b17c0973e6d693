// CPU oracle for the quantized-linear path of BetaDoggo/comfyui-backend-but-rust.
//
// TEST INFRASTRUCTURE ONLY. This file restates, on host cores, the arithmetic of the reference's CUDA
// kernels for the path (activation quantizer, ConvRot rotation, int8 GEMM with fused dequant epilogue,
// W6 decode, quantize-at-load weight packers). It is the checker the parity tests compare the CUDA
// kernels against, and the "host cores" baseline the benchmark reports. The product library never links,
// loads or calls it.
//
// Parity pin: the reference's own tests hold no golden vector for this path ("parity unpinned" by the
// reference). This restatement is pinned instead against the reference's own CUDA kernels compiled for
// sm_100a (oracle/build_ref.sh) and run on a B200: the GPU tests compare all three pairwise.
//
// Every function cites the reference file:line it follows (paths inside the reference project).
// Built with -ffp-contract=off: no fused multiply-add is formed except where fmaf() is written.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

// ---- scalar conversions -------------------------------------------------------------------------
inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// float -> bf16 bits, round to nearest even (what __float2bfloat16_rn does; csrc/common.cuh:27)
inline uint16_t f2bf(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;  // NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float bf2f(uint16_t b) { return u2f((uint32_t)b << 16); }
inline float rnd_bf(float v) { return bf2f(f2bf(v)); }
// float -> half -> float, round to nearest even (csrc/common.cuh:28)
inline uint16_t f2h(float f) { _Float16 h = (_Float16)f; uint16_t b; std::memcpy(&b, &h, 2); return b; }
inline float h2f(uint16_t b) { _Float16 h; std::memcpy(&h, &b, 2); return (float)h; }
inline float rnd_h(float v) { return h2f(f2h(v)); }

enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };  // csrc/common.cuh:15
inline float rnd_t(int dt, float v) { return dt == DT_BF16 ? rnd_bf(v) : dt == DT_F16 ? rnd_h(v) : v; }
inline float ld_t(int dt, const void* p, int64_t i) {
    if (dt == DT_BF16) return bf2f(((const uint16_t*)p)[i]);
    if (dt == DT_F16) return h2f(((const uint16_t*)p)[i]);
    return ((const float*)p)[i];
}
inline void st_t(int dt, void* p, int64_t i, float v) {
    if (dt == DT_BF16) ((uint16_t*)p)[i] = f2bf(v);
    else if (dt == DT_F16) ((uint16_t*)p)[i] = f2h(v);
    else ((float*)p)[i] = v;
}

// fp8 e4m3 (no infinities; 0x7f/0xff are NaN) -> float, exact; csrc/h3.cu:5
inline float e4m3_to_f(uint8_t v) {
    const int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
    float r;
    if (e == 0) r = std::ldexp((float)m, -9);
    else if (e == 15 && m == 7) r = NAN;
    else r = std::ldexp((float)(8 + m), e - 10);
    return s ? -r : r;
}

// ---- activations (csrc/common.cuh:71-95) ----------------------------------------------------------
// expf/tanhf/erff here are the host libm's: results can differ from the CUDA ones in the last fp32 ulp,
// which the tests allow for (at most one int8 step on a small fraction of elements).
inline float silu_f(float x) { return x / (1.f + expf(-x)); }
inline float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
inline float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
// csrc/common.cuh:73-81: tanh through expm1 (accurate near zero) and the soft-capped gated activation built on it
inline float stable_tanh(float x) {
    const float t = expm1f(-2.f * fabsf(x));
    return copysignf(-t / (t + 2.f), x);
}
inline float situ_f(float hidden, float gate) {
    return 4.f * stable_tanh(gate / 4.f) / (1.f + expf(-gate)) * (25.f * stable_tanh(hidden / 25.f));
}
inline float gelu_tanh_f(float x, int contract) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    // nvcc contracts x + k1*x*x*x into an fma in the reference build; `contract` restates that.
    const float inner = contract ? fmaf(k1 * x * x, x, x) : x + k1 * x * x * x;
    const float t = tanhf(k0 * inner);
    return contract ? fmaf(0.5f * x, t, 0.5f * x) : 0.5f * x * (1.f + t);
}

// ---- ConvRot rotation (csrc/common.cuh:99-126; csrc/sd.cu:560-576) -----------------------------------
// One radix-4 stage set over groups of `group` (256: four stages, 64: three) of a row of K floats.
// Each butterfly reads x0..x3 then writes 0.5 * (((+-x0 +- x1) +- x2) +- x3), left to right.
void fht_rows(float* row, int K, int group) {
    const int stages = group == 256 ? 4 : 3;
    for (int g0 = 0; g0 < K; g0 += group) {
        float* v = row + g0;
        for (int st = 0; st < stages; ++st) {
            const int s = 1 << (2 * st);
            for (int r = 0; r < group / 4; ++r) {
                const int i0 = (r / s) * (s << 2) + (r % s);
                const float x0 = v[i0], x1 = v[i0 + s], x2 = v[i0 + 2 * s], x3 = v[i0 + 3 * s];
                v[i0] = 0.5f * (x0 + x1 + x2 - x3);
                v[i0 + s] = 0.5f * (x0 + x1 - x2 + x3);
                v[i0 + 2 * s] = 0.5f * (x0 - x1 + x2 + x3);
                v[i0 + 3 * s] = 0.5f * (-x0 + x1 + x2 + x3);
            }
        }
    }
}

inline int8_t to_i8(float t, float lo) {  // (int8_t)fminf(127, fmaxf(lo, nearbyintf(t))) with CUDA's NaN rules
    float r = nearbyintf(t);
    r = std::isnan(r) ? lo : (r < lo ? lo : r);  // fmaxf(lo, NaN) == lo
    r = r > 127.f ? 127.f : r;
    return (int8_t)r;
}

enum { PRO_PLAIN = 0, PRO_RMS = 1, PRO_GATE = 2, PRO_SWIGLU = 3, PRO_LAYERNORM = 4, PRO_SILU = 5, PRO_GELU = 6,
       PRO_ADALN = 7, PRO_SITU = 8, PRO_LN_MOD = 9, PRO_LN_AFFINE = 10, PRO_GELU_TANH = 11, PRO_SITU_FAST = 13 };  // src/ffi.rs:15-29

}  // namespace

// In-place rotation of M rows of K floats, groups of 256 or 64.
ORC_API void orc_fht_rows(float* x, int64_t M, int K, int group) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) fht_rows(x + m * K, K, group);
}

// Activation quantizer: csrc/kernels.cu:76-259 (quant_rows_kernel) behind gpu_quant_rows (:271-298).
// dtype bf16 or f32; prologues PLAIN, RMS, GATE, SWIGLU, LAYERNORM, SILU, GELU, ADALN, SITU, LN_MOD, LN_AFFINE (with
// norm_b: the gpu_quant_rows_b entry point, kernels.cu:301-314), GELU_TANH. SITU_FAST (hardware tanh and exp
// approximations on the GPU, about 2^-11 relative) is restated with the exact SITU expression.
// The block-wide sums of the norm prologues run in the reference's order: each lane's own elements in
// group order, a shuffle tree over the warp's 32 lanes, then a shuffle tree over the warps
// (csrc/common.cuh:30-52).
// Returns 0, or the reference's negative launcher codes (-1 K%256, -2 K>32768, -3 prologue, -4 dtype).
ORC_API int orc_quant_rows(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                           int64_t up_offset, const float* norm_w, float eps, const void* mod_scale,
                           const void* mod_shift, int8_t* q, float* scales, int M, int K, int rotate, float* out_f,
                           int contract, const float* norm_b) {
    if (K % 256) return -1;
    const int ngroups = K / 256;
    const int nwarps = (ngroups + 3) / 4;
    if (nwarps > 32) return -2;
    if (dtype != DT_BF16 && dtype != DT_F32) return -4;
    switch (prologue) {
        case PRO_PLAIN: case PRO_RMS: case PRO_GATE: case PRO_SWIGLU: case PRO_LAYERNORM: case PRO_SILU:
        case PRO_GELU: case PRO_ADALN: case PRO_GELU_TANH: case PRO_SITU: case PRO_SITU_FAST: case PRO_LN_MOD: break;
        case PRO_LN_AFFINE: if (!norm_w || !norm_b) return -3; break;
        default: return -3;
    }
    const float fmax_t = dtype == DT_BF16 ? 3.38953139e38f : 3.402823466e+38f;  // kernels.cu:49-51
    auto rnd = [dtype](float v) { return rnd_t(dtype, v); };
    // thread (warp, lane) of the reference block owns elements (g<<8) + lane*8 + j for g = warp + gi*nwarps
    auto block_sum = [&](const std::vector<float>& part /* [nwarps*32] per-thread partials */) {
        float wsum[32];
        for (int w = 0; w < nwarps; ++w) {
            float t[32];
            for (int l = 0; l < 32; ++l) t[l] = part[w * 32 + l];
            for (int o = 16; o > 0; o >>= 1) {
                float n[32];
                for (int l = 0; l < 32; ++l) n[l] = t[l] + t[l ^ o];
                std::memcpy(t, n, sizeof(t));
            }
            wsum[w] = t[0];
        }
        float t[32];
        for (int l = 0; l < 32; ++l) t[l] = l < nwarps ? wsum[l] : 0.f;
        for (int o = 16; o > 0; o >>= 1) {
            float n[32];
            for (int l = 0; l < 32; ++l) n[l] = t[l] + t[l ^ o];
            std::memcpy(t, n, sizeof(t));
        }
        return t[0];
    };
#pragma omp parallel
    {
        std::vector<float> v(K), part(nwarps * 32);
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            const int64_t xo = (int64_t)m * x_stride;
            // prologue -> v (kernels.cu:88-182)
            for (int k = 0; k < K; ++k) {
                const float a = ld_t(dtype, x, xo + k);
                switch (prologue) {
                    case PRO_GATE: v[k] = rnd(a * rnd(sigmoid_f(ld_t(dtype, g, (int64_t)m * g_stride + k)))); break;
                    case PRO_SWIGLU: v[k] = rnd(rnd(silu_f(a)) * ld_t(dtype, x, xo + up_offset + k)); break;
                    case PRO_SITU: case PRO_SITU_FAST: v[k] = situ_f(a, ld_t(dtype, x, xo + up_offset + k)); break;  // not rounded here
                    case PRO_SILU: v[k] = rnd(silu_f(a)); break;
                    case PRO_GELU: v[k] = rnd(gelu_f(a)); break;
                    case PRO_GELU_TANH: v[k] = rnd(gelu_tanh_f(a, contract)); break;
                    default: v[k] = a;
                }
            }
            const bool ln = prologue == PRO_LAYERNORM || prologue == PRO_LN_MOD || prologue == PRO_LN_AFFINE;
            if (prologue == PRO_RMS || ln || prologue == PRO_ADALN) {
                auto thread_partials = [&](auto f) {
                    for (int w = 0; w < nwarps; ++w)
                        for (int l = 0; l < 32; ++l) {
                            float ss = 0.f;
                            for (int gi = 0; gi < 4; ++gi) {
                                const int gg = w + gi * nwarps;
                                if (gg >= ngroups) break;
                                for (int j = 0; j < 8; ++j) ss = f(ss, v[(gg << 8) + l * 8 + j]);
                            }
                            part[w * 32 + l] = ss;
                        }
                };
                if (ln) {
                    thread_partials([](float ss, float e) { return ss + e; });
                    const float mean = block_sum(part) / (float)K;
                    for (int k = 0; k < K; ++k) v[k] -= mean;
                }
                // ss += v*v: nvcc forms an fma here in the reference build when contract is set
                if (contract) thread_partials([](float ss, float e) { return fmaf(e, e, ss); });
                else thread_partials([](float ss, float e) { return ss + e * e; });
                const float ss = block_sum(part);
                const float rstd = 1.0f / sqrtf(ss / (float)K + eps);  // rsqrtf on the GPU (<= 2 ulp apart)
                for (int k = 0; k < K; ++k) {
                    float n = v[k] * rstd;
                    if (prologue == PRO_ADALN) {
                        const float ms = ld_t(dtype, mod_scale, k), sh = ld_t(dtype, mod_shift, k);
                        v[k] = rnd(contract ? fmaf(n, 1.f + ms, sh) : n * (1.f + ms) + sh);
                        continue;
                    }
                    if (prologue == PRO_LN_MOD) {   // kernels.cu:40: one rounding after the norm, one after the addcmul
                        const float ms = mod_scale ? ld_t(dtype, mod_scale, k) : 0.f, sh = mod_scale ? ld_t(dtype, mod_shift, k) : 0.f;
                        v[k] = rnd(fmaf(rnd(n), rnd(1.f + ms), sh));
                        continue;
                    }
                    if (prologue == PRO_LN_AFFINE) {   // kernels.cu:41
                        v[k] = rnd(fmaf(n, norm_w[k], norm_b[k]));
                        continue;
                    }
                    if (norm_w) n *= norm_w[k];
                    n = rnd(n);
                    if (mod_scale) {
                        const float a = rnd(1.f + ld_t(dtype, mod_scale, k));
                        // f32 rows: rnd is the identity and nvcc fuses a * n + shift in the reference build
                        if (dtype == DT_F32 && contract) n = fmaf(a, n, ld_t(dtype, mod_shift, k));
                        else n = rnd(rnd(a * n) + ld_t(dtype, mod_shift, k));
                    }
                    v[k] = n;
                }
            }
            if (rotate) fht_rows(v.data(), K, 256);  // kernels.cu:184-222
            if (out_f) {                              // kernels.cu:227-238
                std::memcpy(out_f + (int64_t)m * K, v.data(), sizeof(float) * K);
                continue;
            }
            float amax = 0.f;
            for (int k = 0; k < K; ++k) amax = fmaxf(amax, fabsf(v[k]));
            const float scale = fmaxf(fminf(amax, fmax_t) * (1.f / 127.f), 1.0e-30f);  // kernels.cu:241
            scales[m] = scale;
            const float st = rnd(scale);
            int8_t* qr = q + (int64_t)m * K;
            for (int k = 0; k < K; ++k) qr[k] = to_i8(rnd(rnd(v[k]) / st), -128.f);  // kernels.cu:252-254
        }
    }
    return 0;
}

// fp16 row quantizer, activations and weights at load: csrc/sd.cu:578-606. rotate in {0, 64, 256}.
ORC_API int orc_sd_quant_rows(const void* x, int64_t x_stride, int8_t* q, float* scales, int M, int K, int rotate) {
    if ((rotate != 0 && rotate != 64 && rotate != 256) || (rotate && K % rotate)) return -1;
#pragma omp parallel
    {
        std::vector<float> row(K);
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            for (int k = 0; k < K; ++k) row[k] = h2f(((const uint16_t*)x)[(int64_t)m * x_stride + k]);
            if (rotate) fht_rows(row.data(), K, rotate);
            float mx = 0.f;
            for (int k = 0; k < K; ++k) mx = fmaxf(mx, fabsf(rnd_h(row[k])));
            const float scale = fmaxf(mx, 1e-30f) / 127.f;
            scales[m] = scale;
            const float st = rnd_h(scale) > 0.f ? rnd_h(scale) : scale;
            for (int k = 0; k < K; ++k) q[(int64_t)m * K + k] = to_i8(rnd_h(rnd_h(row[k]) / st), -128.f);
        }
    }
    return 0;
}

// The fp16 quantizer over a row another kernel would have produced (csrc/sd.cu:611-708): mode 1 LayerNorm with f32
// weight and bias (sd_layer_norm_kernel's sums: 256 threads, thread t adds elements t, t + 256, ..., then the block
// tree of csrc/common.cuh:42-55), 2 GEGLU of [M, 2K] (value, gate), 3 head un-padding of [M, heads, dp] to heads * d.
ORC_API int orc_sd_src_quant_rows(int mode, const void* x, int64_t x_stride, const float* w, const float* b, float eps, int heads,
                                  int d, int dp, int8_t* q, float* scales, int M, int K, int rotate) {
    if ((rotate != 0 && rotate != 64 && rotate != 256) || (rotate && K % rotate)) return -1;
    if (mode < 1 || mode > 3) return -3;
    const uint16_t* xh = (const uint16_t*)x;
    auto block_sum256 = [](const float* part) {   // part[256] per-thread sums
        float wsum[8];
        for (int wi = 0; wi < 8; ++wi) {
            float t[32];
            for (int l = 0; l < 32; ++l) t[l] = part[wi * 32 + l];
            for (int o = 16; o > 0; o >>= 1) {
                float n[32];
                for (int l = 0; l < 32; ++l) n[l] = t[l] + t[l ^ o];
                std::memcpy(t, n, sizeof(t));
            }
            wsum[wi] = t[0];
        }
        float t[32];
        for (int l = 0; l < 32; ++l) t[l] = l < 8 ? wsum[l] : 0.f;
        for (int o = 16; o > 0; o >>= 1) {
            float n[32];
            for (int l = 0; l < 32; ++l) n[l] = t[l] + t[l ^ o];
            std::memcpy(t, n, sizeof(t));
        }
        return t[0];
    };
#pragma omp parallel
    {
        std::vector<float> row(K);
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            if (mode == 1) {
                const uint16_t* r = xh + (int64_t)m * x_stride;
                float part[256];
                for (int t = 0; t < 256; ++t) {
                    float sacc = 0.f;
                    for (int k = t; k < K; k += 256) sacc += h2f(r[k]);
                    part[t] = sacc;
                }
                const float mean = block_sum256(part) / (float)K;
                for (int t = 0; t < 256; ++t) {
                    float ss = 0.f;
                    for (int k = t; k < K; k += 256) {
                        const float dd = h2f(r[k]) - mean;
                        ss = fmaf(dd, dd, ss);           // nvcc fuses ss += d * d
                    }
                    part[t] = ss;
                }
                const float rstd = 1.0f / sqrtf(block_sum256(part) / (float)K + eps);   // rsqrtf on the GPU (<= 2 ulp apart)
                for (int k = 0; k < K; ++k) row[k] = rnd_h(fmaf((h2f(r[k]) - mean) * rstd, w[k], b[k]));
            } else if (mode == 2) {
                const uint16_t* r = xh + (int64_t)m * 2 * K;
                for (int k = 0; k < K; ++k) row[k] = rnd_h(h2f(r[k]) * rnd_h(gelu_f(h2f(r[K + k]))));
            } else {
                const uint16_t* r = xh + (int64_t)m * heads * dp;
                for (int k = 0; k < K; ++k) row[k] = h2f(r[(k / d) * dp + k % d]);
            }
            if (rotate) fht_rows(row.data(), K, rotate);
            float mx = 0.f;
            for (int k = 0; k < K; ++k) mx = fmaxf(mx, fabsf(rnd_h(row[k])));
            const float scale = fmaxf(mx, 1e-30f) / 127.f;
            scales[m] = scale;
            const float st = rnd_h(scale) > 0.f ? rnd_h(scale) : scale;
            for (int k = 0; k < K; ++k) q[(int64_t)m * K + k] = to_i8(rnd_h(rnd_h(row[k]) / st), -128.f);
        }
    }
    return 0;
}

// GroupNorm (no SiLU) of x [N, P, C] half fused into the fp16 quantizer of its pixels' rows (csrc/sd.cu:198-233, :244-255,
// :710-724). Group sums: per (group, split of the pixels) 256 per-thread float sums over values t, t + 256, ... and the
// block tree, added in double; mean and 1/sqrt(var + eps) in double, then float.
ORC_API int orc_sd_gn_quant_rows(const void* x, const float* w, const float* b, int N, int64_t P, int C, int G, float eps,
                                 int8_t* q, float* scales, int rotate) {
    if (G <= 0 || C % G) return -1;
    if ((rotate != 0 && rotate != 64 && rotate != 256) || (rotate && C % rotate)) return -1;
    const uint16_t* xh = (const uint16_t*)x;
    const int per = C / G;
    const int64_t want = P * per / 4096;
    const int splits = want < 1 ? 1 : want > 64 ? 64 : (int)want;
    const double cnt = (double)P * per;
    auto tree256 = [](const float* part) {
        float wsum[8];
        for (int wi = 0; wi < 8; ++wi) {
            float t[32];
            for (int l = 0; l < 32; ++l) t[l] = part[wi * 32 + l];
            for (int o = 16; o > 0; o >>= 1) { float n2[32]; for (int l = 0; l < 32; ++l) n2[l] = t[l] + t[l ^ o]; std::memcpy(t, n2, sizeof(t)); }
            wsum[wi] = t[0];
        }
        float t[32];
        for (int l = 0; l < 32; ++l) t[l] = l < 8 ? wsum[l] : 0.f;
        for (int o = 16; o > 0; o >>= 1) { float n2[32]; for (int l = 0; l < 32; ++l) n2[l] = t[l] + t[l ^ o]; std::memcpy(t, n2, sizeof(t)); }
        return t[0];
    };
    std::vector<float> mean_f((size_t)N * G), rstd_f((size_t)N * G);
#pragma omp parallel for schedule(static)
    for (int ng = 0; ng < N * G; ++ng) {
        const int n = ng / G, g = ng % G;
        const int64_t base = (int64_t)n * P * C + g * per;
        double su = 0.0, sq = 0.0;
        for (int split = 0; split < splits; ++split) {
            const int64_t p0 = P * split / splits, p1 = P * (split + 1) / splits, count = (p1 - p0) * per;
            float ps[256], pq[256];
            for (int t = 0; t < 256; ++t) {
                float s1 = 0.f, s2 = 0.f;
                for (int64_t i = t; i < count; i += 256) {
                    const float v = h2f(xh[base + (p0 + i / per) * C + (int)(i % per)]);
                    s1 += v;
                    s2 = fmaf(v, v, s2);
                }
                ps[t] = s1, pq[t] = s2;
            }
            su += (double)tree256(ps);
            sq += (double)tree256(pq);
        }
        const double mean = su / cnt;
        const double var = fmax(fma(-mean, mean, sq / cnt), 0.0);
        mean_f[ng] = (float)mean;
        rstd_f[ng] = (float)(1.0 / sqrt(var + (double)eps));
    }
    const int64_t M = (int64_t)N * P;
#pragma omp parallel
    {
        std::vector<float> row(C);
#pragma omp for schedule(static)
        for (int64_t m = 0; m < M; ++m) {
            const int n = (int)(m / P);
            for (int c = 0; c < C; ++c) {
                const int ng = n * G + c / per;
                row[c] = rnd_h(fmaf((h2f(xh[m * C + c]) - mean_f[ng]) * rstd_f[ng], w[c], b[c]));
            }
            if (rotate) fht_rows(row.data(), C, rotate);
            float mx = 0.f;
            for (int c = 0; c < C; ++c) mx = fmaxf(mx, fabsf(rnd_h(row[c])));
            const float scale = fmaxf(mx, 1e-30f) / 127.f;
            scales[m] = scale;
            const float st = rnd_h(scale) > 0.f ? rnd_h(scale) : scale;
            for (int c = 0; c < C; ++c) q[m * C + c] = to_i8(rnd_h(rnd_h(row[c]) / st), -128.f);
        }
    }
    return 0;
}

namespace {
// float -> fp8 e4m3 bits, round to nearest even, saturating to +-448 (what __nv_cvt_float_to_fp8(x, __NV_SATFINITE,
// __NV_E4M3) returns); NaN -> 0x7f.
inline uint8_t f_to_e4m3(float x) {
    if (std::isnan(x)) return 0x7f;
    const uint8_t sign = std::signbit(x) ? 0x80 : 0;
    const float a = fabsf(x);
    if (a >= 448.f) return sign | 0x7e;
    if (a < 0.015625f) return sign | (uint8_t)nearbyintf(a * 512.f);   // denormals: steps of 2^-9 (8 rounds up into the normals)
    int e;
    const float m = frexpf(a, &e);                  // a = m 2^e, m in [0.5, 1)
    int q = (int)nearbyintf(m * 16.f);              // 4 significant bits: 8..16
    int ex = e - 1;
    if (q == 16) q = 8, ++ex;
    const int bits = ((ex + 7) << 3) | (q - 8);
    return sign | (uint8_t)(bits > 0x7e ? 0x7e : bits);
}
inline float w6_level(int i, float s) { return fminf(127.f, fmaxf(-127.f, nearbyintf((float)(i - 31) * s))); }
inline uint32_t pcg_hash(uint32_t x);
}  // namespace

// W6A8 packer, csrc/vendor/w6a8_requant.cu:59-154 and :228-257 (gpu_w6_requant: bf16 input, G = 32, always stochastic).
// packed [N, 3K/4], s_rel [N, K/32] e4m3 bits, s_channel [N].
ORC_API int orc_w6_requant(const void* w, uint8_t* packed, uint8_t* s_rel, float* s_channel, int64_t N, int K, uint64_t seed) {
    if (K % 256) return -1;
    const int groups = K / 32;
    const uint32_t key = (uint32_t)seed ^ (uint32_t)(seed >> 32);
#pragma omp parallel
    {
        std::vector<float> row(K), gstep(groups);
#pragma omp for schedule(static)
        for (int64_t n = 0; n < N; ++n) {
            for (int k = 0; k < K; ++k) row[k] = ld_t(DT_BF16, w, n * K + k);
            fht_rows(row.data(), K, 256);
            for (int k = 0; k < K; ++k) row[k] = rnd_bf(row[k]);
            float amax_row = 0.f;
            for (int g = 0; g < groups; ++g) {
                const float* v = row.data() + g * 32;
                float amax = 0.f;
                for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
                float gs = fmaxf(amax / 31.f, 1e-8f), inv = 1.f / gs;
                for (int it = 0; it < 2; ++it) {
                    float num = 0.f, den = 0.f;
                    for (int i = 0; i < 32; ++i) {
                        const float q = fminf(31.f, fmaxf(-31.f, nearbyintf(v[i] * inv)));
                        num = fmaf(v[i], q, num);       // nvcc fuses num += w * q and den += q * q
                        den = fmaf(q, q, den);
                    }
                    gs = fmaxf(num / fmaxf(den, 1e-8f), 1e-8f);
                    inv = 1.f / gs;
                }
                gstep[g] = gs;
                for (int i = 0; i < 32; ++i)
                    amax_row = fmaxf(amax_row, fabsf(fminf(31.f, fmaxf(-31.f, nearbyintf(v[i] * inv))) * gs));
            }
            const float sc = fmaxf(amax_row / 127.f, 1e-8f), inv_sc = 1.f / sc;
            s_channel[n] = sc;
            uint8_t* prow = packed + n * (int64_t)(K / 4 * 3);
            std::memset(prow, 0, (size_t)K / 4 * 3);
            for (int g = 0; g < groups; ++g) {
                const uint8_t sb = f_to_e4m3(gstep[g] / sc);
                s_rel[n * groups + g] = sb;
                const float s = e4m3_to_f(sb), inv_s = 1.f / fmaxf(s, 1e-30f);
                for (int i = 0; i < 32; ++i) {
                    const int e = g * 32 + i;
                    const float t = row[e] * inv_sc;
                    int pos = (int)nearbyintf((ceilf(t) - 0.5f) * inv_s) + 31;
                    pos = std::min(std::max(pos, 0), 63);
                    while (pos > 0 && w6_level(pos - 1, s) >= t) --pos;
                    while (pos < 63 && w6_level(pos, s) < t) ++pos;
                    const int l = std::min(std::max(pos - 1, 0), 61);
                    const float level_lo = w6_level(l, s);
                    const uint32_t h = pcg_hash((uint32_t)(n * (int64_t)K + e) ^ key);
                    const float u = (float)(h >> 8) * (1.0f / 16777216.0f);
                    const float thr = fmaf(u, w6_level(l + 1, s) - level_lo, level_lo);   // fused in the reference build
                    const uint32_t code = (uint32_t)std::min(l + (t > thr ? 1 : 0), 62) + 1u;
                    prow[e >> 1] |= (uint8_t)((code & 15u) << (4 * (e & 1)));
                    prow[K / 2 + (e >> 2)] |= (uint8_t)(((code >> 4) & 3u) << (2 * (e & 3)));
                }
            }
        }
    }
    return 0;
}

namespace {
inline uint32_t pcg_hash(uint32_t x) {  // csrc/kernels.cu:1356-1360
    const uint32_t state = x * 747796405u + 2891336453u;
    const uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
    return (word >> 22u) ^ word;
}
}  // namespace

// Weight [N,K] (f32 or bf16) -> R256 -> row scale -> int8; seed 0 = nearest-even, else PCG-hash stochastic
// rounding: csrc/kernels.cu:1362-1389 (convrot_requant_kernel), :1409-1420 (gpu_convrot_requant).
ORC_API int orc_convrot_requant(int dtype, const void* x, int8_t* q, float* s, int64_t N, int K, uint64_t seed) {
    if (K % 256) return -1;
    const float fmax_t = dtype == DT_BF16 ? 3.38953139e38f : 3.402823466e+38f;
#pragma omp parallel
    {
        std::vector<float> row(K);
#pragma omp for schedule(static)
        for (int64_t m = 0; m < N; ++m) {
            for (int k = 0; k < K; ++k) row[k] = ld_t(dtype, x, m * K + k);
            fht_rows(row.data(), K, 256);
            float amax = 0.f;
            for (int k = 0; k < K; ++k) amax = fmaxf(amax, fabsf(row[k]));
            const float scale = fmaxf(fminf(amax, fmax_t) * (1.f / 127.f), 1.0e-30f);
            s[m] = scale;
            const float st = rnd_t(dtype, scale);
            for (int k = 0; k < K; ++k) {
                const float scaled = rnd_t(dtype, rnd_t(dtype, row[k]) / st);
                if (seed == 0) { q[m * K + k] = to_i8(scaled, -128.f); continue; }
                const uint64_t key = (uint64_t)(m * K + k) + seed;
                const uint32_t folded = (uint32_t)key ^ (uint32_t)(key >> 32);
                const float noise = (float)(pcg_hash(folded) >> 8) * 0x1.0p-24f;
                // bf16: the sum is a bf16 add of the two bf16-rounded terms (kernels.cu:1341-1343)
                const float sum = dtype == DT_BF16 ? rnd_bf(rnd_bf(scaled) + rnd_bf(noise)) : scaled + noise;
                float v = floorf(sum);
                v = std::isnan(v) ? -128.f : (v < -128.f ? -128.f : v);
                q[m * K + k] = (int8_t)(v > 127.f ? 127.f : v);
            }
        }
    }
    return 0;
}

// int8 ConvRot weight -> original basis (f32 or bf16): csrc/kernels.cu:1345-1354, :1393-1405.
ORC_API int orc_convrot_dequant(int dtype, const int8_t* q, const float* s, void* out, int64_t N, int K) {
    if (K % 256) return -1;
#pragma omp parallel
    {
        std::vector<float> row(K);
#pragma omp for schedule(static)
        for (int64_t m = 0; m < N; ++m) {
            for (int k = 0; k < K; ++k) row[k] = (float)q[m * K + k] * s[m];
            fht_rows(row.data(), K, 256);
            for (int k = 0; k < K; ++k) st_t(dtype, out, m * K + k, row[k]);
        }
    }
    return 0;
}

// int8 [N,K] * scale[n] -> f32: csrc/kernels.cu:330-343.
ORC_API int orc_dequant_i8(const int8_t* q, const float* s, float* out, int64_t N, int64_t K) {
    if (K % 4) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) out[n * K + k] = (float)q[n * K + k] * s[n];
    return 0;
}

// int8 ConvRot embedding rows -> f32 rows holding bf16 values: csrc/kernels.cu:622-638.
ORC_API int orc_embed_dequant(const int8_t* q, const float* s, float* out, int M, int K, int rotate) {
    if (!rotate || K % 256) return -1;
#pragma omp parallel
    {
        std::vector<float> row(K);
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            for (int k = 0; k < K; ++k) row[k] = (float)q[(int64_t)m * K + k] * s[m];
            fht_rows(row.data(), K, 256);
            for (int k = 0; k < K; ++k) out[(int64_t)m * K + k] = rnd_bf(row[k]);
        }
    }
    return 0;
}

// W6 two-plane decode to the int8 grid the GEMM reads: csrc/h3.cu:11-46.
// Row n: K/2 nibble bytes (element e in byte e/2, low nibble when e is even), then K/4 bytes holding the
// top two bits of four consecutive elements at bit offsets 0,2,4,6; s_rel one e4m3 per G columns.
ORC_API int orc_w6_decode(const uint8_t* q, const uint8_t* s_rel, int8_t* out, int64_t N, int K, int G) {
    if (K % 32 || G % 16) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* row = q + n * (K * 3 / 4);
        for (int e = 0; e < K; ++e) {
            const uint8_t lo = row[e / 2];
            const unsigned nib = (e & 1) ? (lo >> 4) : (lo & 15);
            const unsigned top = (row[K / 2 + e / 4] >> (2 * (e % 4))) & 3u;
            const unsigned c = nib | (top << 4);
            const float sc = e4m3_to_f(s_rel[n * (K / G) + e / G]);
            float r = nearbyintf(((float)c - 32.f) * sc);
            r = std::isnan(r) ? -127.f : (r < -127.f ? -127.f : r);
            out[n * K + e] = (int8_t)(r > 127.f ? 127.f : r);
        }
    }
    return 0;
}

// ---- int8 GEMM, int32 accumulate: the product csrc/vendor/cutlass_gemm_int8.cu:65-120 computes -------
// A [M,K] row-major, W [N,K] row-major, acc[m,n] = sum_k A[m,k]*W[n,k] (exact; |acc| < 2^31 for K < 131072).
namespace {
__attribute__((target_clones("arch=icelake-server", "avx2", "default")))
void gemm_rows(const int8_t* A, const int8_t* W, int32_t* acc, int64_t m0, int64_t m1, int64_t N, int64_t K) {
    // 4 rows of A against one row of W at a time; plain loops the compiler vectorizes.
    for (int64_t m = m0; m < m1; m += 4) {
        const int mr = (int)std::min<int64_t>(4, m1 - m);
        for (int64_t n = 0; n < N; ++n) {
            const int8_t* w = W + n * K;
            int32_t s[4] = {0, 0, 0, 0};
            for (int r = 0; r < mr; ++r) {
                const int8_t* a = A + (m + r) * K;
                int32_t t = 0;
                for (int64_t k = 0; k < K; ++k) t += (int32_t)a[k] * (int32_t)w[k];
                s[r] = t;
            }
            for (int r = 0; r < mr; ++r) acc[(m + r) * N + n] = s[r];
        }
    }
}
}  // namespace

ORC_API int orc_int8_gemm_acc(const int8_t* A, const int8_t* W, int32_t* acc, int64_t M, int64_t N, int64_t K) {
    const int64_t blk = 16;
    const int64_t nb = (M + blk - 1) / blk;
#pragma omp parallel for schedule(dynamic)
    for (int64_t b = 0; b < nb; ++b) gemm_rows(A, W, acc, b * blk, std::min(M, (b + 1) * blk), N, K);
    return 0;
}

// Fused dequant epilogue: csrc/vendor/cutlass_gemm_int8.cu:84-95 (plain) and :143-161 (residual), behind
// gpu_int8_gemm / gpu_int8_gemm_residual (csrc/gemm.cu:123-140).
//   y = out_rn( float(acc)*xs[m]*ws[n] + bias[n] )          bias in the output dtype, nullable
//   D = out_rn( float(y)*rscale[n] + resid[m,n] )           when rscale/resid are given
//   D = out_rn( act(float(y)) )                             when act != 0 (1 gelu-tanh, 2 silu, 3 gelu-erf):
//       what the reference's next quantizer prologue computes from y (csrc/kernels.cu:121-130)
// contract bit 0: t1*ws + bias as one fma; bit 1: y*rscale + resid as one fma; bit 2: gelu-tanh contraction.
// Which forms the reference binary uses is decided by comparing against it on the GPU.
ORC_API int orc_epilogue(const int32_t* acc, const float* xs, const float* ws, const void* bias, const void* rscale,
                         const void* resid, void* D, int64_t M, int64_t N, int out_dt, int act, int contract) {
    if (out_dt < 0 || out_dt > 2) return -200;
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            const float t0 = (float)acc[m * N + n] * xs[m];
            const float b = bias ? ld_t(out_dt, bias, n) : 0.f;
            float y = rnd_t(out_dt, (contract & 1) ? fmaf(t0, ws[n], b) : t0 * ws[n] + b);
            if (rscale) {
                const float rs = ld_t(out_dt, rscale, n), rr = ld_t(out_dt, resid, m * N + n);
                y = rnd_t(out_dt, (contract & 2) ? fmaf(y, rs, rr) : y * rs + rr);
            } else if (act == 1) y = rnd_t(out_dt, gelu_tanh_f(y, (contract >> 2) & 1));
            else if (act == 2) y = rnd_t(out_dt, silu_f(y));
            else if (act == 3) y = rnd_t(out_dt, gelu_f(y));
            st_t(out_dt, D, m * N + n, y);
        }
    }
    return 0;
}

// The whole linear on host cores (quantized GEMM + epilogue), the timed CPU baseline.
ORC_API int orc_int8_gemm(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias,
                          const void* rscale, const void* resid, void* D, int64_t M, int64_t N, int64_t K, int out_dt,
                          int act, int contract) {
    if (M == 0 || N == 0) return 0;
    std::vector<int32_t> acc((size_t)M * N);
    orc_int8_gemm_acc(A, W, acc.data(), M, N, K);
    return orc_epilogue(acc.data(), xs, ws, bias, rscale, resid, D, M, N, out_dt, act, contract);
}

// Overrides the OpenMP thread count (launchers such as torchrun export OMP_NUM_THREADS=1).
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
