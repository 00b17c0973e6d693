/* C ABI of libb200_qlinear.so / libb200_qlinear.a: the quantized-linear path of BetaDoggo/comfyui-backend-but-rust for sm_100a.
 *
 * Every function keeps the name, argument order and meaning of the symbol the reference's Rust side declares in
 * src/ffi.rs and its CUDA side defines (cited per function as file:line inside the reference project), so the
 * Rust code links against this library unchanged for these calls.
 *
 * Conventions (reference: csrc/common.cuh:12,15,128; src/ffi.rs:336-355):
 *   - return 0 on success; a negative launcher code on a rejected argument; a positive cudaError_t otherwise
 *   - every pointer is a DEVICE pointer owned by the caller unless stated; nothing is allocated for the caller
 *   - `stream` is a cudaStream_t; calls only enqueue work on it and never synchronise
 *   - dtype / out_dt codes: 0 = f32, 1 = f16, 2 = bf16
 *   - no C++ exception crosses this boundary; nothing is printed
 */
#ifndef GPU_KERNELS_H
#define GPU_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { GPU_DT_F32 = 0, GPU_DT_F16 = 1, GPU_DT_BF16 = 2 }; /* src/ffi.rs:11-13 */

/* quantizer prologues, src/ffi.rs:15-29 */
enum {
    GPU_PRO_PLAIN = 0, GPU_PRO_RMS = 1, GPU_PRO_GATE = 2, GPU_PRO_SWIGLU = 3, GPU_PRO_LAYERNORM = 4, GPU_PRO_SILU = 5,
    GPU_PRO_GELU = 6, GPU_PRO_ADALN = 7, GPU_PRO_SITU = 8, GPU_PRO_LN_MOD = 9, GPU_PRO_LN_AFFINE = 10,
    GPU_PRO_GELU_TANH = 11, GPU_PRO_LN_AFFINE_SILU = 12, GPU_PRO_SITU_FAST = 13
};

/* ---- kernel 1: activation quantizer ------------------------------------------------------------------- */

/* Row prologue -> optional ConvRot rotation (R256 per 256-wide group when rotate != 0) -> per-row absmax int8.
 * x [M, x_stride] bf16 or f32, rows 16-byte aligned; q int8 [M, K]; scales f32 [M].
 * Errors: -1 K % 256 != 0, -2 K > 32768, -3 prologue not available, -4 dtype, -5 a row of x (or of g, or the
 * second half at up_offset), q or out does not start on a 16-byte boundary (the reference's 16-byte loads fault there).
 * Replaces csrc/kernels.cu:271-298 (declared at src/ffi.rs:74). */
int gpu_quant_rows(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                   int64_t up_offset, const float* norm_w, float eps, const void* mod_scale, const void* mod_shift,
                   int8_t* q, float* scales, int M, int K, int rotate, void* stream);

/* gpu_quant_rows for the LayerNorm prologues that carry a bias: LN_AFFINE (norm_w, norm_b [K] f32) and LN_MOD
 * (mod_scale, mod_shift [K] bf16). bf16 input only (-4), other prologues -3.
 * Replaces csrc/kernels.cu:301-314 (src/ffi.rs:143). */
int gpu_quant_rows_b(int dtype, int prologue, const void* x, int64_t x_stride, const float* norm_w, const float* norm_b,
                     float eps, const void* mod_scale, const void* mod_shift, int8_t* q, float* scales, int M, int K,
                     int rotate, void* stream);

/* Prologue + rotation, rotated rows written as f32 [M, K] (weight-only int8 layers' activation side).
 * Replaces csrc/kernels.cu:316-327 (src/ffi.rs:35). */
int gpu_rotate_rows_f32(int prologue, const float* x, int64_t x_stride, int64_t up_offset, const float* norm_w, float eps,
                        float* out, int M, int K, void* stream);

/* fp16 rows (SD/SDXL activations, and fp16 weights at load) -> rotate 0 | 64 | 256 -> int8 + f32 row scale.
 * Errors: -1 bad rotate. Replaces csrc/sd.cu:599-606 (src/ffi.rs:246). */
int gpu_sd_quant_rows(const void* x, int64_t x_stride, int8_t* q, float* scales, int M, int K, int rotate, void* stream);

/* gpu_sd_quant_rows over a row that another kernel of the reference would have written in half first, computed here
 * as that kernel computes it (same order of additions, same rounding to half) and quantized without the intermediate
 * in memory: LayerNorm with f32 weight and bias; GEGLU of in [M, 2I] (value, then gate); head un-padding of
 * src [M, H, dp] to [M, H*d]. Errors as gpu_sd_quant_rows. Replace csrc/sd.cu:690-724 (src/ffi.rs:247-253).
 * gpu_sd_group_norm_quant_rows: GroupNorm (no SiLU) of x [N, P, C] with G groups, then the quantizer of its N*P rows of
 * C values; sums = scratch of N*G*2 doubles + 16 bytes (cleared here). -1 also for C % G != 0 or G > 256. */
int gpu_sd_ln_quant_rows(const void* x, int64_t x_stride, const float* w, const float* b, float eps, int8_t* q,
                         float* scales, int M, int K, int rotate, void* stream);
int gpu_sd_geglu_quant_rows(const void* in, int8_t* q, float* scales, int M, int I, int rotate, void* stream);
int gpu_sd_unpad_quant_rows(const void* src, int8_t* q, float* scales, int M, int H, int d, int dp, int rotate,
                            void* stream);
int gpu_sd_group_norm_quant_rows(const void* x, const float* w, const float* b, void* sums, int N, int64_t P, int C, int G,
                                 float eps, int8_t* q, float* scales, int rotate, void* stream);

/* ---- kernels 2 + 3: int8 GEMM mainloop with the fused dequant epilogue -------------------------------- */

/* D[M,N] = out( (A[M,K] . W[N,K]^T) * xs[m] * ws[n] + bias[n] ).  A, W int8 row-major (K contiguous), 16-byte
 * aligned with K % 16 == 0 for the tensor-core kernel (K % 8 == 0 or bases off a 16-byte boundary: a slower CUDA-core
 * kernel, same results); xs f32 [M]; ws f32 [N]; bias [N] in the OUTPUT dtype or NULL; D [M,N] row-major.
 * M == 0, N == 0 or K == 0 succeed without work. Errors: -200 bad out_dt or K % 8 != 0 (the reference's "no tile
 * configuration"; -201 from the residual form), -203 descriptor.
 * Replaces csrc/gemm.cu:123-129 over csrc/vendor/cutlass_gemm_int8.cu:373-388 (src/ffi.rs:38). */
int gpu_int8_gemm(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias, void* D,
                  int64_t M, int64_t N, int64_t K, int out_dt, void* stream);

/* D = out( resid[m,n] + rscale[n] * out( acc * xs[m] * ws[n] + bias[n] ) ); rscale [N] and resid [M,N] in the
 * output dtype, both required (-201 when NULL, or when K == 0); D may alias resid.
 * Replaces csrc/gemm.cu:131-140 over csrc/vendor/cutlass_gemm_int8.cu:348-371 (src/ffi.rs:39). */
int gpu_int8_gemm_residual(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias,
                           const void* rscale, const void* resid, void* D, int64_t M, int64_t N, int64_t K, int out_dt,
                           void* stream);

/* New (the reference applies the activation in the NEXT quantizer's prologue, csrc/kernels.cu:121-130):
 * D = out( act( out( acc * xs[m] * ws[n] + bias[n] ) ) ), act 0 none, 1 gelu-tanh, 2 silu, 3 gelu-erf, so that
 * "this call, then a PLAIN quantizer" equals "gpu_int8_gemm, then the quantizer with that prologue". -204 bad act. */
int gpu_int8_gemm_act(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias, void* D,
                      int64_t M, int64_t N, int64_t K, int out_dt, int act, void* stream);

/* New: the MLP's "GEMM -> quantizer with activation prologue and rotation" (src/qwen21.rs:378-417; the quantizer is
 * csrc/kernels.cu:76-259 with PRO_GELU_TANH / PRO_SILU / PRO_GELU and rotate = 1) with the activation AND the R256 rotation
 * moved into the GEMM's epilogue, which holds one rotation group (256 columns) of every row in tensor memory:
 *   gpu_int8_gemm_act_rot   D[m, :] = bf16( R256( act( bf16( acc * xs[m] * ws[n] + bias[n] ) ) ) )   (bf16 only), and
 *                           amax_part [N / 64, M] f32 (part-major): partial row maxima of the unrounded rotated values
 *                           (four per 256-column group), sign bit set when a NaN was among them;
 *   gpu_quant_rows_rotated  xr = that D, amax_part -> q [M, K] int8, scales [M] f32.
 * The pair gives the codes and scales of gpu_int8_gemm followed by gpu_quant_rows(prologue = the activation, rotate = 1),
 * bit for bit. N % 256 == 0, K % 16 == 0, operands 16-byte aligned, act 1..3 (-208 otherwise); second call: K % 256 == 0
 * (-1), xr and q 16-byte aligned (-5). */
int gpu_int8_gemm_act_rot(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias, void* D,
                          float* amax_part, int64_t M, int64_t N, int64_t K, int act, void* stream);
int gpu_quant_rows_rotated(const void* xr, const float* amax_part, int8_t* q, float* scales, int M, int K, void* stream);

/* No counterpart in the reference. gpu_int8_gemm for hosts that must not allocate device memory once they run (an
 * engine that manages the card inside a fixed budget of its own, a latency-critical thread): small-output, long-K
 * problems (at most 16 tiles of 256 x 256 outputs) are cut along K, and the scratch the slices meet in is a
 * 4,259,840-byte array inside the loaded module instead of an allocation. Returns -205 when the problem needs more than
 * the array holds (use gpu_int8_gemm then); other codes as gpu_int8_gemm. Makes no cudaMalloc / cudaFree or other
 * allocating call. The first call on each device looks up the array's device address: issue it before any stream
 * capture. The array is shared by every call and keeps the previous call's contents; each call clears what it uses on
 * `stream`, so calls must not overlap on the GPU (serialise streams that use it). */
int gpu_int8_gemm_noalloc(const int8_t* A, const int8_t* W, const float* xs, const float* ws, const void* bias, void* D,
                          int64_t M, int64_t N, int64_t K, int out_dt, void* stream);

/* New, for tests: the raw int32 accumulators D[m,n] = sum_k A[m,k] * W[n,k] that the fused forms never expose. */
int gpu_int8_gemm_acc_i32(const int8_t* A, const int8_t* W, int32_t* D, int64_t M, int64_t N, int64_t K, void* stream);

/* New: the W6A8 linear straight from the packed weight. The reference expands Wq6 to int8 in a scratch buffer with
 * gpu_w6_decode (csrc/h3.cu:11-46) and calls gpu_int8_gemm on that copy (src/h3.rs:1208-1216); these take the packed rows
 * Wq6 [N, 3K/4] (nibble plane, then 2-bit plane) and the e4m3 group scales s_rel [N, K/G] and expand them in shared
 * memory on the way to the tensor cores. Results equal gpu_w6_decode followed by gpu_int8_gemm[_residual] bit for bit;
 * ws is the per-output-channel scale (s_channel). K % 128 == 0, Wq6 16-byte and s_rel 4-byte aligned (-202), G == 32
 * (-206). gpu_w6a8_gemm_act applies the activation of gpu_int8_gemm_act to the rounded output (the FFN-up linear with
 * GELU of the W6A8 video DiT; act 1 gelu-tanh, 2 silu, 3 gelu-erf, -204 otherwise). gpu_w6a8_gemm_acc_i32 (for tests)
 * returns the raw int32 accumulators. */
int gpu_w6a8_gemm(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, const float* xs, const float* ws,
                  const void* bias, void* D, int64_t M, int64_t N, int64_t K, int G, int out_dt, void* stream);
int gpu_w6a8_gemm_residual(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, const float* xs, const float* ws,
                           const void* bias, const void* rscale, const void* resid, void* D, int64_t M, int64_t N,
                           int64_t K, int G, int out_dt, void* stream);
int gpu_w6a8_gemm_act(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, const float* xs, const float* ws,
                      const void* bias, void* D, int64_t M, int64_t N, int64_t K, int G, int out_dt, int act, void* stream);
int gpu_w6a8_gemm_acc_i32(const int8_t* A, const uint8_t* Wq6, const uint8_t* s_rel, int32_t* D, int64_t M, int64_t N,
                          int64_t K, int G, void* stream);

/* New, for tensor-parallel linears whose K columns are split across devices (the reference is single-device):
 * two-pass quantization around a max-reduction of the row maxima between the devices. Pass 1 writes the local row
 * maxima (after prologue and rotation) to amax [M]; pass 2 quantizes with the given maxima. Same argument meaning
 * and error codes as gpu_quant_rows. With the reduced maxima the codes equal the single-device ones bit for bit. */
int gpu_quant_rows_amax(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                        int64_t up_offset, float* amax, int M, int K, int rotate, void* stream);
int gpu_quant_rows_scaled(int dtype, int prologue, const void* x, int64_t x_stride, const void* g, int64_t g_stride,
                          int64_t up_offset, const float* amax, int8_t* q, float* scales, int M, int K, int rotate,
                          void* stream);

/* New: the dequant epilogue alone over int32 accumulators [M, N] already in global memory (e.g. partial products of a
 * row-parallel linear summed by a reduce-scatter): the arithmetic of gpu_int8_gemm (resid == NULL, act == 0),
 * gpu_int8_gemm_act (act != 0) or gpu_int8_gemm_residual (rscale and resid given; D may alias resid). */
int gpu_int8_epilogue(const int32_t* acc, const float* xs, const float* ws, const void* bias, const void* rscale,
                      const void* resid, void* D, int64_t M, int64_t N, int out_dt, int act, void* stream);

/* New: the weight-only int8 linear of the text encoders in one call. The reference runs gpu_rotate_rows_f32
 * (csrc/kernels.cu:316-327), dequantizes the whole weight with gpu_dequant_i8 (:330-343) and calls an fp32 GEMM with beta 0
 * or 1 (src/te.rs:493-511); this computes out[M,N] = beta * out + R256(prologue(x)) . (Wq * ws[n])^T on the bf16 tensor
 * cores: Wq [N,K] int8 widens to bf16 exactly, the rotated f32 rows go as two bf16 terms (hi + lo) in two accumulating
 * passes, f32 accumulators. prologue PLAIN, RMS (norm_w, eps) or SWIGLU (up_offset) as for gpu_rotate_rows_f32 (-3).
 * a_scratch >= 4*M*K bytes, w_scratch >= 2*N*K bytes, 16-byte aligned (-202); beta 0 or 1 (-207); K % 256 == 0 (-1).
 * Result: within 1e-5 of the largest output of the fp32 flow (tests state the bound). */
int gpu_wo8_linear(int prologue, const float* x, int64_t x_stride, int64_t up_offset, const float* norm_w, float eps,
                   const int8_t* Wq, const float* ws, float* out, float beta, void* a_scratch, void* w_scratch, int M, int N,
                   int K, void* stream);

/* New (tensor parallelism): the tail of a row-parallel linear whose dequantized partial outputs were summed across
 * devices: out[:, n0:n0+Nc] = T(T(y + bias[n0:n0+Nc]) + resid[:, n0:n0+Nc]); y [M, Nc] contiguous, resid / out [M, ld]
 * (out may alias resid), bias and resid nullable, all in the activation dtype dt. Nc, n0, ld multiples of 8 and
 * pointers 16-byte aligned (-202). No counterpart in the reference (single device). */
int gpu_bias_residual_add(const void* y, const void* bias, const void* resid, void* out, int64_t M, int64_t Nc, int64_t ld,
                          int64_t n0, int dt, void* stream);

/* New (tensor parallelism): gpu_int8_gemm* launches that follow occupy at most `clusters` CTA pairs (0 = all of the
 * device's SM pairs, the default), so that a collective running on another stream finds SMs free. Process-wide;
 * returns the previous value. No counterpart in the reference. */
int gpu_int8_gemm_set_cluster_limit(int clusters);

/* W6A8: q [N, 3K/4] u8 (per row K/2 nibble bytes then K/4 bytes of top bits), s_rel [N, K/G] fp8-e4m3 ->
 * out int8 [N, K] = clamp(rint((code - 32) * s_rel), +-127). -1 when K % 32 or G % 16.
 * Replaces csrc/h3.cu:40-46 (src/ffi.rs:121). */
int gpu_w6_decode(const void* q, const void* s_rel, void* out, int64_t N, int K, int G, void* stream);

/* The W6A8 packer: bf16 weight [N, K] -> R256 -> packed [N, 3K/4] (nibble plane, then 2-bit plane), s_rel e4m3 [N, K/32],
 * s_channel f32 [N]; group steps by two least-squares rounds, levels drawn by stochastic rounding keyed by seed and
 * element index. -1: K % 256. Replaces csrc/vendor/w6a8_requant.cu:246-257 (src/ffi.rs:132). */
int gpu_w6_requant(const void* weight, void* packed, void* s_rel, void* s_channel, int64_t N, int K, uint64_t seed,
                   void* stream);

/* ---- kernel 4: quantize-at-load weight packers and their inverses ------------------------------------- */

/* x [N, K] f32 or bf16 -> R256 -> q int8 [N, K] + s f32 [N]; seed 0 rounds to nearest even, any other seed rounds
 * stochastically (PCG hash of element index + seed). -1 K % 256, -4 dtype.
 * Replaces csrc/kernels.cu:1409-1420 (src/ffi.rs:119). */
int gpu_convrot_requant(int dtype, const void* x, void* q, void* s, int64_t N, int K, uint64_t seed, void* stream);

/* q int8 [N, K] (rotated), s [N] -> out [N, K] f32 or bf16 in the original basis.
 * Replaces csrc/kernels.cu:1393-1405 (src/ffi.rs:118). */
int gpu_convrot_dequant(int dtype, const void* q, const void* s, void* out, int64_t N, int K, void* stream);

/* out[n, k] = q[n, k] * s[n] as f32; -1 when K % 4. Replaces csrc/kernels.cu:337-343 (src/ffi.rs:37). */
int gpu_dequant_i8(const int8_t* q, const float* s, float* out, int64_t N, int64_t K, void* stream);

/* int8 ConvRot embedding rows -> f32 rows holding bf16 values; -1 unless rotate.
 * Replaces csrc/kernels.cu:633-638 (src/ffi.rs:82). */
int gpu_embed_dequant(const int8_t* q, const float* s, float* out, int M, int K, int rotate, void* stream);

/* Windows video-memory budget query the Rust side imports unconditionally (src/cuda.rs:136-153; the reference
 * defines it in csrc/wddm.cu). HOST pointers. Always returns non-zero here: no budget is known. */
int gpu_wddm_budget(uint64_t* budget, uint64_t* usage);

/* ---- library housekeeping (new) ------------------------------------------------------------------------ */

/* Reads and clears the device status word of the current device (synchronises it). *status (HOST pointer) is 0
 * unless a kernel gave up one of its bounded waits (1-5: which wait). */
int gpu_kernels_status(int* status);

#ifdef __cplusplus
}
#endif
#endif /* GPU_KERNELS_H */
