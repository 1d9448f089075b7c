// Per-(token, head) group quantisation shared by the append and the exchange-pack kernels.
//
// A group of 128 channels is held by 8 lanes, 16 channels each.  Codes are bit-identical to
// QuantizedCompressor._quantize_tensor (core/single/module/pikv_compression.py:965-1006) on the
// [1,128] slice, i.e. to rint(fl(fl(x / scale) + zp)), but without a division per element: the
// correctly rounded quotient comes from one reciprocal per lane and two exact-remainder fma
// refinements, and adding 1.5 * 2^23 rounds to the nearest integer (ties to even) while leaving the
// integer in the low mantissa bits.  Groups outside the range where that is exact (denormal or huge
// scales, the multi-million zero point of a constant group) take the IEEE division.
#pragma once
#include "common.cuh"

namespace pikv {

constexpr float QG_MAGIC = 12582912.0f;          // 1.5 * 2^23
constexpr int QG_MAGIC_BITS = 0x4B400000;

template <typename TIn>
__device__ __forceinline__ void qg_load16(const TIn* p, float (&x)[16]);
template <>
__device__ __forceinline__ void qg_load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[16]) {
    // the lane's two 16-byte halves share one 32-byte sector: let the first load allocate it in L1
    uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    uint4 b = __ldg(reinterpret_cast<const uint4*>(p + 8));
    bf16x2_to_f32(a.x, x[0], x[1]);   bf16x2_to_f32(a.y, x[2], x[3]);
    bf16x2_to_f32(a.z, x[4], x[5]);   bf16x2_to_f32(a.w, x[6], x[7]);
    bf16x2_to_f32(b.x, x[8], x[9]);   bf16x2_to_f32(b.y, x[10], x[11]);
    bf16x2_to_f32(b.z, x[12], x[13]); bf16x2_to_f32(b.w, x[14], x[15]);
}
template <>
__device__ __forceinline__ void qg_load16<float>(const float* p, float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 a = ld_stream_16(p + 4 * i);
        x[4 * i + 0] = __uint_as_float(a.x); x[4 * i + 1] = __uint_as_float(a.y);
        x[4 * i + 2] = __uint_as_float(a.z); x[4 * i + 3] = __uint_as_float(a.w);
    }
}

// min / max of the 128-channel group this lane belongs to (8 consecutive lanes)
__device__ __forceinline__ void qg_group_minmax(const float (&x)[16], float& mn, float& mx) {
    mn = x[0];
    mx = x[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
}

__device__ __forceinline__ uint32_t qg_pack4_s8(int n0, int n1, int n2, int n3) {
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(n3), "r"(n2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(n1), "r"(n0), "r"(hi));
    return out;
}
__device__ __forceinline__ uint32_t qg_pack4_u8(int n0, int n1, int n2, int n3) {
    uint32_t hi, out;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(n3), "r"(n2), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(n1), "r"(n0), "r"(hi));
    return out;
}

// fp32 -> bf16 bits, round to nearest even, integer pipe only (finite inputs)
__device__ __forceinline__ uint16_t qg_bf16_bits(float x) {
    const uint32_t u = __float_as_uint(x);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// Symmetric 8-bit codes of this lane's 16 channels, the hot case.  x / scale is bracketed by
// x * inv_lo and x * inv_hi (inv = 1/scale moved 2^-20 either way, far more than the 2^-24 of the
// reciprocal and of the reference's division); adding 1.5 * 2^23 inside the fma rounds each to the
// nearest integer, ties to even, exactly like rint.  When both ends give the same integer, so
// does the reference; the xor of the two bit patterns accumulates the exceptions, and a thread
// with any redoes its 16 channels with the IEEE division.  The integer is the low byte of the
// float's bit pattern, so four codes are packed with three byte permutes; only +128 (x = +absmax,
// 127.5 rounding to even) needs the clamp.
__device__ __forceinline__ void qg_quantize16_s8(const float (&x)[16], float mn, float mx, QParams& qp, uint32_t (&w)[4]) {
    qp = quant_params(mn, mx, -128, 127, true);
    const float inv = __frcp_rn(qp.scale);
    const float inv_lo = inv * 0.99999905f, inv_hi = inv * 1.00000095f;
    uint32_t t[16];
    uint32_t diff = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float tl = __fmaf_rn(x[i], inv_lo, QG_MAGIC);
        const float th = __fmaf_rn(x[i], inv_hi, QG_MAGIC);
        diff |= __float_as_uint(tl) ^ __float_as_uint(th);
        t[i] = __float_as_uint(fminf(tl, QG_MAGIC + 127.0f));
    }
    if (diff != 0u || !(inv < 3.0e38f)) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float q = fminf(fmaxf(rintf(__fdiv_rn(x[i], qp.scale)), -128.f), 127.f);
            t[i] = (uint32_t)(int)q;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = __byte_perm(t[4 * i], t[4 * i + 1], 0x0040);
        const uint32_t hi = __byte_perm(t[4 * i + 2], t[4 * i + 3], 0x0040);
        w[i] = __byte_perm(lo, hi, 0x5410);
    }
}

typedef unsigned long long qg_f2;   // two fp32 in one 64-bit register pair
__device__ __forceinline__ qg_f2 qg_pk(float lo, float hi) {
    qg_f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ qg_f2 qg_pku(uint32_t lo, uint32_t hi) {
    qg_f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void qg_unpku(qg_f2 v, uint32_t& lo, uint32_t& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ qg_f2 qg_fma2(qg_f2 a, qg_f2 b, qg_f2 c) {
    qg_f2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ qg_f2 qg_mul2(qg_f2 a, qg_f2 b) {
    qg_f2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ qg_f2 qg_add2(qg_f2 a, qg_f2 b) {
    qg_f2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Quantise this lane's 16 channels.  Returns the packed codes in w (4 words for 8 bits, 2 for 4).
template <int BITS, bool SYM>
__device__ __forceinline__ void qg_quantize16(const float (&x)[16], float mn, float mx, QParams& qp, uint32_t (&w)[4]) {
    if (BITS == 8 && SYM) {
        qg_quantize16_s8(x, mn, mx, qp, w);
        return;
    }
    constexpr int QMIN = SYM ? -(1 << (BITS - 1)) : 0;
    constexpr int QMAX = SYM ? (1 << (BITS - 1)) - 1 : (1 << BITS) - 1;
    qp = quant_params(mn, mx, QMIN, QMAX, SYM);
    // rint(fl(fl(x / scale) + zp)), the reference's sequence, without a division per element: the correctly
    // rounded quotient from y = RN(1 / scale) and two exact-remainder refinements (see the 8-bit symmetric
    // routine below), the fp32 add of zp, and 1.5 * 2^23 added to round to the nearest integer, ties to
    // even; two elements per instruction.  Outside the range where the remainders are exact and the sum
    // fits the trick (tiny / huge scales, the multi-million zero point of a constant group) every
    // element takes the IEEE division.
    const float amax = fmaxf(fabsf(mn), fabsf(mx));
    const bool fast = qp.scale > 1.0e-30f && qp.scale < 1.0e30f && amax < 1.0e30f && fabsf(qp.zp) < 1048576.0f &&
                      amax < 1048576.0f * qp.scale;
    int n[16];
    if (fast) {
        const float y = __frcp_rn(qp.scale);
        const qg_f2 y2 = qg_pk(y, y), ns2 = qg_pk(-qp.scale, -qp.scale), magic2 = qg_pk(QG_MAGIC, QG_MAGIC);
        const qg_f2 zp2 = qg_pk(qp.zp, qp.zp);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const qg_f2 x2 = qg_pk(x[2 * i], x[2 * i + 1]);
            qg_f2 q = qg_mul2(x2, y2);
            qg_f2 r = qg_fma2(ns2, q, x2);
            q = qg_fma2(r, y2, q);
            r = qg_fma2(ns2, q, x2);
            q = qg_fma2(r, y2, q);                       // RN(x / scale)
            q = qg_add2(q, zp2);                         // RN(. + zp)
            q = qg_add2(q, magic2);                      // rint, integer in the low mantissa bits
            uint32_t lo, hi;
            qg_unpku(q, lo, hi);
            n[2 * i] = (int)lo - QG_MAGIC_BITS;
            n[2 * i + 1] = (int)hi - QG_MAGIC_BITS;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) n[i] = (int)rintf(__fadd_rn(__fdiv_rn(x[i], qp.scale), qp.zp));
    }
    if (BITS == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = SYM ? qg_pack4_s8(n[4 * i], n[4 * i + 1], n[4 * i + 2], n[4 * i + 3])
                       : qg_pack4_u8(n[4 * i], n[4 * i + 1], n[4 * i + 2], n[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!SYM) {
                // codes 0..15: four per word by the saturating byte pack, then neighbouring bytes merged
                // into nibbles (low nibble = even channel) and the four merged bytes gathered
                int c[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) c[j] = min(n[8 * i + j], 15);      // the pack below saturates at 0
                uint32_t a = qg_pack4_u8(c[0], c[1], c[2], c[3]), b = qg_pack4_u8(c[4], c[5], c[6], c[7]);
                a |= a >> 4;
                b |= b >> 4;
                w[i] = __byte_perm(a, b, 0x6420);
            } else {
                uint32_t v = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) v |= (uint32_t)(min(max(n[8 * i + j], QMIN), QMAX) & 0xf) << (4 * j);
                w[i] = v;
            }
        }
        w[2] = w[3] = 0;
    }
}

// ---- bf16 in, symmetric 8-bit out ------------------------------------------------------------
// Statistics on the raw bf16 pairs: one packed max and one packed min per word give max |x| and
// "all 128 channels equal" (the reference's x_max == x_min case, which moves x_max up by 1e-5).
//
// Codes: bf16 inputs make x / scale land exactly on a .5 tie in about one element in 400 (ratios of
// small integers), and the group's max sits on 127.5 by construction, so the code depends on how
// the reference's fp32 division rounds: the quotient has to be the correctly rounded one.  It is
// formed without a per-element reciprocal: y = RN(1/scale) once per lane, then
//   q = x*y ; r = fma(-scale, q, x) ; q = fma(r, y, q) ; r = fma(-scale, q, x) ; q = fma(r, y, q)
// (two exact-remainder refinements: the second one is correctly rounded, Markstein), and
// q + 1.5*2^23 rounds to the nearest integer, ties to even, exactly like rint.  All six steps are
// packed two elements per instruction (fma/mul/add.f32x2).
// the reference's own sequence, one IEEE division per element; kept out of line because it is rare
static __device__ __noinline__ uint4 qg_exact_s8_bf16(uint4 a, uint4 b, float scale) {
    const uint32_t ww[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t acc = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int e = 4 * i + c;
            const float x = __uint_as_float((e & 1) ? (ww[e >> 1] & 0xffff0000u) : (ww[e >> 1] << 16));
            const int q = (int)fminf(fmaxf(rintf(__fdiv_rn(x, scale)), -128.f), 127.f);
            acc |= ((uint32_t)q & 0xffu) << (8 * c);
        }
        out[i] = acc;
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

__device__ __forceinline__ void qg_quantize16_s8_bf16(const uint4& a, const uint4& b, QParams& qp, uint32_t (&w)[4]) {
    const uint32_t ww[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    // signed max and min of the packed pairs: max |x| is the larger magnitude of the two, and the group is
    // constant exactly when they are equal as numbers (+0 and -0 included)
    uint32_t hi2 = ww[0], lo2 = ww[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        asm("max.bf16x2 %0, %0, %1;" : "+r"(hi2) : "r"(ww[i]));
        asm("min.bf16x2 %0, %0, %1;" : "+r"(lo2) : "r"(ww[i]));
    }
    float gmax = fmaxf(__uint_as_float(hi2 << 16), __uint_as_float(hi2 & 0xffff0000u));
    float gmin = fminf(__uint_as_float(lo2 << 16), __uint_as_float(lo2 & 0xffff0000u));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
        gmin = fminf(gmin, __shfl_xor_sync(0xffffffffu, gmin, o));
    }
    const bool all_equal = gmax == gmin;
    float abs_max = fmaxf(fabsf(gmax), fabsf(gmin));
    if (all_equal) {
        // every channel holds the same value c (or +-0): x_min = c, x_max = c + 1e-5
        const float c = gmin;
        abs_max = fmaxf(fabsf(c), fabsf(__fadd_rn(c, 1e-5f)));
    }
    qp.scale = __fdiv_rn(__fmul_rn(2.0f, abs_max), 255.0f);
    qp.zp = 0.0f;
    if (!(abs_max > 1.0e-30f && abs_max < 1.0e30f)) {
        // denormal / overflowing scale: the refinement's remainders are not exact there
        const uint4 r = qg_exact_s8_bf16(a, b, qp.scale);
        w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
        return;
    }
    const float y = __frcp_rn(qp.scale);
    const qg_f2 y2 = qg_pk(y, y), ns2 = qg_pk(-qp.scale, -qp.scale), magic2 = qg_pk(QG_MAGIC, QG_MAGIC);
    uint32_t t[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const qg_f2 x2 = qg_pku(ww[i] << 16, ww[i] & 0xffff0000u);
        qg_f2 q = qg_mul2(x2, y2);
        qg_f2 r = qg_fma2(ns2, q, x2);
        q = qg_fma2(r, y2, q);
        r = qg_fma2(ns2, q, x2);
        q = qg_fma2(r, y2, q);                       // RN(x / scale)
        q = qg_add2(q, magic2);                      // rint, integer in the low mantissa bits
        uint32_t lo, hi;
        qg_unpku(q, lo, hi);
        t[2 * i] = (uint32_t)min((int)lo, QG_MAGIC_BITS + 127);     // +128 (x = +absmax) clamps to 127
        t[2 * i + 1] = (uint32_t)min((int)hi, QG_MAGIC_BITS + 127);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = __byte_perm(t[4 * i], t[4 * i + 1], 0x0040);
        const uint32_t hi = __byte_perm(t[4 * i + 2], t[4 * i + 3], 0x0040);
        w[i] = __byte_perm(lo, hi, 0x5410);
    }
}

// Load and quantisation of one group slice (16 channels of this lane), split so that a kernel can
// issue the loads of its next item before it quantises the current one.  All 32 lanes must call
// quant() together (the statistics shuffle across the 8 lanes of a group).
template <typename TIn, int BITS, bool SYM>
struct GroupQuant {
    struct Raw { float x[16]; };
    static __device__ __forceinline__ void load(const TIn* src, Raw& r) { qg_load16<TIn>(src, r.x); }
    static __device__ __forceinline__ void quant(const Raw& r, QParams& qp, uint32_t (&w)[4]) {
        float mn, mx;
        qg_group_minmax(r.x, mn, mx);
        qg_quantize16<BITS, SYM>(r.x, mn, mx, qp, w);
    }
};
// bf16 in, any other format out: the raw words stay packed while an item waits in the software pipeline (half the
// registers of sixteen floats per tensor), the group's minimum and maximum come from packed bf16 min / max (exact:
// they only select), and the floats exist only inside quant().
template <int BITS, bool SYM>
struct GroupQuant<__nv_bfloat16, BITS, SYM> {
    struct Raw { uint4 a, b; };
    static __device__ __forceinline__ void load(const __nv_bfloat16* src, Raw& r) {
        r.a = __ldg(reinterpret_cast<const uint4*>(src));
        r.b = __ldg(reinterpret_cast<const uint4*>(src + 8));
    }
    static __device__ __forceinline__ void quant(const Raw& r, QParams& qp, uint32_t (&w)[4]) {
        const uint32_t ww[8] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w};
        uint32_t hi2 = ww[0], lo2 = ww[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) {
            asm("max.bf16x2 %0, %0, %1;" : "+r"(hi2) : "r"(ww[i]));
            asm("min.bf16x2 %0, %0, %1;" : "+r"(lo2) : "r"(ww[i]));
        }
        float mx = fmaxf(__uint_as_float(hi2 << 16), __uint_as_float(hi2 & 0xffff0000u));
        float mn = fminf(__uint_as_float(lo2 << 16), __uint_as_float(lo2 & 0xffff0000u));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        float x[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) bf16x2_to_f32(ww[i], x[2 * i], x[2 * i + 1]);
        qg_quantize16<BITS, SYM>(x, mn, mx, qp, w);
    }
};
template <>
struct GroupQuant<__nv_bfloat16, 8, true> {
    struct Raw { uint4 a, b; };
    static __device__ __forceinline__ void load(const __nv_bfloat16* src, Raw& r) {
        // the lane's two 16-byte halves share one 32-byte sector: the first load allocates it in L1
        r.a = __ldg(reinterpret_cast<const uint4*>(src));
        r.b = __ldg(reinterpret_cast<const uint4*>(src + 8));
    }
    static __device__ __forceinline__ void quant(const Raw& r, QParams& qp, uint32_t (&w)[4]) {
        qg_quantize16_s8_bf16(r.a, r.b, qp, w);
    }
};

}  // namespace pikv
