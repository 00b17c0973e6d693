// Expansion of W6A8 codes to int8, shared by the decode kernel (weight_pack.cu) and the fused GEMM (gemm_w6.inl).
// Storage (the reference's, csrc/h3.cu:8-37, csrc/vendor/w6a8_requant.cu:128-151): per weight row K/2 bytes of low nibbles
// (element e in byte e/2, even e in the low nibble), then K/4 bytes holding the top two bits of four consecutive
// elements; one fp8-e4m3 scale per 32 columns; the int8 value is clamp(rint((code - 32) * scale), +-127).
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

// One scale group: 32 codes (16 bytes of nibbles l, top bits ha for elements 0-15 and hb for 16-31, scale byte sb) ->
// 32 int8 in element order (o[0..7]).
// A word of nibbles holds 8 elements, the even ones in the low nibbles; its 16 top bits hold one 2-bit field per
// element. Masked with 0x3333 they are, as they stand, a byte-permute selector (one index 0..3 per nibble) for the
// even elements, and shifted right by two for the odd ones, so one permute of a 4-byte table turns four fields into
// the four high nibbles. With a scale of exactly 1 the table holds the high nibble of code - 32 as a signed byte
// (E, F, 0, 1) and the result is final; otherwise it holds code bits 5:4 and the bytes go through half-precision
// arithmetic two at a time: 1024 + code by setting exponent bits, one fused multiply-add with -1056 * s (exact while
// that constant is finite), clamp where 32 * |s| can pass 127, rint by adding 1536, low bytes gathered by a permute.
__device__ __forceinline__ void w6_group(const uint4 l, uint32_t ha, uint32_t hb, uint32_t sb, uint32_t (&o)[8]) {
    const uint32_t lw[4] = {l.x, l.y, l.z, l.w};
    const uint32_t hv[2] = {ha, hb};
    // The three forms are chosen per warp, not per lane: lanes hold different rows with different scales, and a branch that
    // splits the warp costs the sum of its sides. The general form is right for every scale, the clamped one too.
    if (__all_sync(0xffffffffu, sb == 0x38u)) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t h = hv[w >> 1] >> (16 * (w & 1));
            const uint32_t te = __byte_perm(0x1000F0E0u, 0u, h & 0x3333u), to = __byte_perm(0x1000F0E0u, 0u, (h >> 2) & 0x3333u);
            const uint32_t de = (lw[w] & 0x0F0F0F0Fu) | te, dd = ((lw[w] >> 4) & 0x0F0F0F0Fu) | to;
            o[2 * w] = __byte_perm(de, dd, 0x5140);        // e0 o0 e1 o1
            o[2 * w + 1] = __byte_perm(de, dd, 0x7362);    // e2 o2 e3 o3
        }
        return;
    }
    const __half2 s2 = __half2half2(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)sb, __NV_E4M3)));
    const __half2 magic = __float2half2_rn(1536.f);
    const bool clamp = __any_sync(0xffffffffu, (sb & 0x7fu) >= 0x48u);   // some |s| >= 4 (or NaN): 32 * |s| can pass 127
    const __half2 c2 = __hmul2(__float2half2_rn(-1056.f), s2);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t h = hv[w >> 1] >> (16 * (w & 1));
        const uint32_t te = __byte_perm(0x30201000u, 0u, h & 0x3333u), to = __byte_perm(0x30201000u, 0u, (h >> 2) & 0x3333u);
        const uint32_t ce = (lw[w] & 0x0F0F0F0Fu) | te, co = ((lw[w] >> 4) & 0x0F0F0F0Fu) | to;
        uint32_t p[4] = {__byte_perm(ce, 0x64646464u, 0x4140), __byte_perm(co, 0x64646464u, 0x4140),     // (e0,e2) (e1,e3)
                         __byte_perm(ce, 0x64646464u, 0x4342), __byte_perm(co, 0x64646464u, 0x4342)};    // (e4,e6) (e5,e7)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 g = *reinterpret_cast<__half2*>(&p[i]);
            if (!clamp) {
                g = __hfma2(g, s2, c2);
            } else {
                g = __hmul2(__hsub2(g, __float2half2_rn(1056.f)), s2);
                g = __hmin2(__hmax2(g, __float2half2_rn(-127.f)), __float2half2_rn(127.f));
            }
            g = __hadd2(g, magic);
            p[i] = *reinterpret_cast<uint32_t*>(&g);
        }
        o[2 * w] = __byte_perm(p[0], p[1], 0x6240);
        o[2 * w + 1] = __byte_perm(p[2], p[3], 0x6240);
    }
}

