// The dequant epilogue's arithmetic, shared by the GEMM kernels (one element at a time here; the tensor-core kernel
// applies the same operations eight columns at a time).
//   t0 = float(acc) * xs;  y = out(fma(t0, ws, bias));  residual: fma(y, rscale, resid);  activation: act(y)
// The caller rounds the returned value to the output type when it stores it.
// Reference: csrc/vendor/cutlass_gemm_int8.cu:84-95 and :143-161 (nvcc fuses both multiply-adds there).
#pragma once

#include "common.cuh"

// EPI_ACT computes the activation; EPI_ACT_LUT (tensor-core kernel, bf16 outputs) reads bf16(act(x)) from a table instead;
// EPI_ACT_ROT does that and rotates each 256-column group of the row (R256) before the store
enum EpiMode { EPI_PLAIN = 0, EPI_RESID = 1, EPI_ACT = 2, EPI_ACC = 3, EPI_ACT_LUT = 4, EPI_ACT_ROT = 5 };
enum Act { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_GELU_ERF = 3 };

template <typename OutT, int EPI>
__device__ __forceinline__ float epilogue1(int acc, float xs, float ws, float bias, float rscale, float resid, int act) {
    const float t0 = __fmul_rn(__int2float_rn(acc), xs);
    float v = rnd<OutT>(__fmaf_rn(t0, ws, bias));
    if (EPI == EPI_RESID) v = __fmaf_rn(v, rscale, resid);
    else if (EPI == EPI_ACT) v = act == ACT_GELU_TANH ? gelu_tanh_f(v) : act == ACT_SILU ? silu_f(v) : gelu_f(v);
    return v;
}

// Arguments of the few-rows kernel (gemm_skinny.cu); launched from the GEMM entry points in gemm_i8.cu.
struct SkinnyParams {
    const int8_t* A;     // [M, K]
    const int8_t* W;     // [N, K]
    const float* xs;
    const float* ws;
    const void* bias;
    const void* rscale;
    const void* resid;
    void* D;
    int M, N, K;
    int act;
};
// Helpers shared between the translation units (a namespace of their own: the static archive exports them).
namespace b200q {
// quant_rows.cu: table of bf16(act(x)) over all bf16 x for Act code `act`, built on first use (on `st`)
int act_lut_ptr(int act, cudaStream_t st, const uint16_t** out);
// quant_rows.cu: the quantizer's status word (non-zero after a staging wait ran out), read and cleared
int quant_status_read_clear(int* out);
// quant_rows.cu: gpu_rotate_rows_f32's prologue + rotation with the rows written as two bf16 terms [M, K] each
int rotate_rows_split(int prologue, const float* x, int64_t x_stride, int64_t up_offset, const float* norm_w, float eps, void* hi,
                      void* lo, int M, int K, cudaStream_t st);
// quant_rows.cu: the fp16 row quantizer on the register kernel; false when the shape is outside what it takes
bool sd_quant_rows_fast(const void* x, int64_t x_stride, int8_t* q, float* scales, int M, int K, int rotate, cudaStream_t st, int* rc);
bool skinny_gemm_applies(int64_t M, int64_t N, int64_t K);
int launch_skinny_gemm(int epi, const SkinnyParams& p, int out_dt, int sms, cudaStream_t st);
// gemm_skinny.cu: the CUDA-core kernel for operands TMA cannot address (K % 16 != 0, bases off a 16-byte boundary)
int launch_generic_gemm(int epi, const SkinnyParams& p, int out_dt, cudaStream_t st);
}  // namespace b200q
using namespace b200q;
