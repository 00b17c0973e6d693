/* A host program in plain C against include/gpu_kernels.h: no Python, no torch. It quantizes a few activation rows
 * (gpu_quant_rows, no rotation), multiplies them with an int8 weight (gpu_int8_gemm_acc_i32, gpu_int8_gemm with f32
 * output) and checks the int32 accumulators exactly and the dequantized outputs to float rounding against loops
 * written here. Exit code 0 = all equal. Built and run by tests/test_c_abi_gpu.py. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_runtime_api.h>

#include "gpu_kernels.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("cuda error %d at line %d\n", (int)e_, __LINE__); return 2; } } while (0)
#define RC(x) do { int r_ = (x); if (r_ != 0) { printf("launcher code %d at line %d\n", r_, __LINE__); return 3; } } while (0)

static uint32_t rng = 12345u;
static uint32_t next_u32(void) { rng = rng * 1664525u + 1013904223u; return rng; }

int main(void) {
    enum { M = 70, K = 512, N = 136 };
    float* x = (float*)malloc(sizeof(float) * M * K);
    int8_t* w = (int8_t*)malloc(N * K);
    float* ws = (float*)malloc(sizeof(float) * N);
    float* bias = (float*)malloc(sizeof(float) * N);
    for (int i = 0; i < M * K; ++i) x[i] = (float)((int)(next_u32() >> 8) % 2001 - 1000) / 250.0f;
    for (int i = 0; i < N * K; ++i) w[i] = (int8_t)((int)(next_u32() >> 8) % 255 - 127);
    for (int n = 0; n < N; ++n) ws[n] = 1e-3f + (float)(next_u32() >> 8) / 16777216.0f * 1e-3f, bias[n] = (float)(n % 7) * 0.25f - 0.5f;

    float *dx, *dscales, *dws, *dbias, *dout;
    int8_t *dq, *dw;
    int32_t* dacc;
    CK(cudaMalloc((void**)&dx, sizeof(float) * M * K));
    CK(cudaMalloc((void**)&dq, M * K));
    CK(cudaMalloc((void**)&dscales, sizeof(float) * M));
    CK(cudaMalloc((void**)&dw, N * K));
    CK(cudaMalloc((void**)&dws, sizeof(float) * N));
    CK(cudaMalloc((void**)&dbias, sizeof(float) * N));
    CK(cudaMalloc((void**)&dacc, sizeof(int32_t) * M * N));
    CK(cudaMalloc((void**)&dout, sizeof(float) * M * N));
    CK(cudaMemcpy(dx, x, sizeof(float) * M * K, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dw, w, N * K, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dws, ws, sizeof(float) * N, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dbias, bias, sizeof(float) * N, cudaMemcpyHostToDevice));

    /* dtype 0 = f32, prologue 0 = PLAIN, rotate 0; stream 0 */
    RC(gpu_quant_rows(0, 0, dx, K, NULL, 0, 0, NULL, 0.f, NULL, NULL, dq, dscales, M, K, 0, NULL));
    RC(gpu_int8_gemm_acc_i32(dq, dw, dacc, M, N, K, NULL));
    RC(gpu_int8_gemm(dq, dw, dscales, dws, dbias, dout, M, N, K, 0, NULL));
    int status = -1;
    RC(gpu_kernels_status(&status));
    if (status != 0) { printf("kernel status %d\n", status); return 4; }

    int8_t* q = (int8_t*)malloc(M * K);
    float* scales = (float*)malloc(sizeof(float) * M);
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * M * N);
    float* out = (float*)malloc(sizeof(float) * M * N);
    CK(cudaMemcpy(q, dq, M * K, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(scales, dscales, sizeof(float) * M, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(acc, dacc, sizeof(int32_t) * M * N, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(out, dout, sizeof(float) * M * N, cudaMemcpyDeviceToHost));

    int bad = 0;
    for (int m = 0; m < M; ++m) {   /* the quantizer: scale = max(amax / 127, 1e-30), q = clamp(rint(x / scale)) */
        float amax = 0.f;
        for (int k = 0; k < K; ++k) amax = fmaxf(amax, fabsf(x[m * K + k]));
        const float scale = fmaxf(amax * (1.f / 127.f), 1e-30f);
        if (scale != scales[m]) ++bad;
        for (int k = 0; k < K; ++k) {
            float t = nearbyintf(x[m * K + k] / scale);
            t = t < -128.f ? -128.f : t > 127.f ? 127.f : t;
            if ((int8_t)t != q[m * K + k]) ++bad;
        }
    }
    if (bad) { printf("quantizer: %d mismatches\n", bad); return 5; }
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            int32_t a = 0;
            for (int k = 0; k < K; ++k) a += (int32_t)q[m * K + k] * (int32_t)w[n * K + k];
            if (a != acc[m * N + n]) ++bad;
            const float want = fmaf((float)a * scales[m], ws[n], bias[n]);   /* the epilogue's fused form */
            if (want != out[m * N + n]) ++bad;
        }
    if (bad) { printf("gemm: %d mismatches\n", bad); return 6; }
    printf("abi smoke ok: %d x %d x %d\n", M, K, N);
    return 0;
}
