// Generic quantized kernels (NCHW, any geometry).  Exact int32 accumulation; requantisation in
// fp32 with the operation order documented in include/zant_b200.h — each step is an explicitly
// rounded intrinsic so the compiler cannot fuse or reorder it.
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "geometry.hpp"

namespace zb {

__device__ __forceinline__ int rne_clamped(float v) {
    // nearest-even of v clamped to [-512, 511]; fmaxf/fminf drop a NaN operand
    v = fminf(fmaxf(v, -512.0f), 511.0f);
    return __float2int_rn(v);
}

// QuantizeLinear's rne(clamp(x / scale, lo, hi)) without the division on the common path.
// q = rint(clamp(x * r, lo, hi)) with r = fl(1 / scale) is the wanted integer unless x / scale lies within a few units
// in the last place of a rounding boundary (k + 0.5) or of a clamp bound.  The residual e = fma(-q, scale, x) is the
// exact x - q * scale rounded once, so |e| < h with h a little below scale / 2 proves that x / scale lies strictly inside
// (q - 0.5, q + 0.5); a q at a clamp bound is proved by the sign of e alone (the true quotient is beyond the bound or
// inside the last half-step).  Everything else - about one value in a few thousand - takes the correctly rounded division.
// The reference formula rounds the fp32 quotient d = fl(x / scale), so the proof needs a margin of half a unit in the
// last place of d around the boundaries: with |d| < 256 that is below 8e-6, and h leaves 1e-4.
// `lo` and `hi` are integers in [-255, 255] (the clamp of the reference formula with the zero point folded in).  A scale
// that is not positive and finite disables the fast path (h = -1 and unreachable bounds).
struct QuantFast { float scale, r, h, lo, hi, klo, khi; };

__host__ __device__ inline QuantFast quant_fast(float scale, float lo, float hi) {
    QuantFast q;
    const bool usable = scale > 0.0f && scale < 3.0e38f && (1.0f / scale) < 3.0e38f && lo >= -255.0f && hi <= 255.0f;
    q.scale = scale; q.r = usable ? 1.0f / scale : 0.0f; q.h = usable ? scale * 0.4999f : -1.0f; q.lo = lo; q.hi = hi;
    q.klo = usable ? lo : -1.0e30f; q.khi = usable ? hi : 1.0e30f;
    return q;
}

__device__ __forceinline__ int quantize_fast(float x, const QuantFast& q) {
    const float t = __fmul_rn(x, q.r);
    const float c = fminf(fmaxf(t, q.lo), q.hi);         // a NaN becomes lo, as in the division form
    const float k = rintf(c);
    const float e = __fmaf_rn(-k, q.scale, x);
    const bool proved = fabsf(e) < q.h || (k == q.khi && e > 0.0f) || (k == q.klo && e < 0.0f);
    if (proved) return (int)k;
    return __float2int_rn(fminf(fmaxf(__fdiv_rn(x, q.scale), q.lo), q.hi));
}

template <bool U8> __device__ __forceinline__ int sat_q(int t) {
    return U8 ? min(max(t, 0), 255) : min(max(t, -128), 127);
}

struct Requant {
    float y_scale; int y_zp; int act;   // zant_qact
    // Optional 256-entry table (device memory) applied to the finished output code, indexed by the unsigned
    // view of the byte: an element-wise operator between two quantized tensors (LeakyRelu, a Relu or Clip that
    // changes scale) folded into the producer.  Exact by construction: the producer computes the very code the
    // separate operator would have read.
    const uint8_t* lut = nullptr;
};

__device__ __forceinline__ int lut1(const uint8_t* lut, int code) { return (int)__ldg(lut + (code & 255)); }
// the same from a copy of the table in shared memory (64 words over 32 banks: cheap next to divergent global loads)
__device__ __forceinline__ uint32_t lut4_smem(const uint8_t* lut, uint32_t pk) {
    return (uint32_t)lut[pk & 255u] | ((uint32_t)lut[(pk >> 8) & 255u] << 8) | ((uint32_t)lut[(pk >> 16) & 255u] << 16) | ((uint32_t)lut[pk >> 24] << 24);
}
// four packed codes through the table
__device__ __forceinline__ uint32_t lut4(const uint8_t* lut, uint32_t pk) {
    return (uint32_t)__ldg(lut + (pk & 255u)) | ((uint32_t)__ldg(lut + ((pk >> 8) & 255u)) << 8) |
           ((uint32_t)__ldg(lut + ((pk >> 16) & 255u)) << 16) | ((uint32_t)__ldg(lut + (pk >> 24)) << 24);
}

template <bool YU8>
__device__ __forceinline__ int requant_one(int acc, float M, const Requant& r) {
    const float v = __fmul_rn(__int2float_rn(acc), M);
    int t = sat_q<YU8>(rne_clamped(v) + r.y_zp);
    if (r.act != ZANT_QACT_NONE) {
        t = max(t, sat_q<YU8>(r.y_zp));
        if (r.act == ZANT_QACT_RELU6) t = min(t, sat_q<YU8>(rne_clamped(__fdiv_rn(6.0f, r.y_scale)) + r.y_zp));
    }
    if (r.lut) { t = lut1(r.lut, t); if (!YU8) t = (int)(int8_t)t; }
    return t;
}

// ---------------------------------------------------------------------------- lean int8 requantisation
// Fast form of requant_one for int8 outputs with zero point 0 and a positive finite multiplier
// (the host checks both).  rni(float(acc) * M) saturates at the int32 range and the pack
// instruction saturates to [-128,127]; for zero point 0 that equals
// sat(rne(clamp(v,-512,511)) + 0) for every v, so the results are bit-identical.
__device__ __forceinline__ int rq_round(int acc, float M) { return __float2int_rn(__fmul_rn(__int2float_rn(acc), M)); }

// ReLU / ReLU6 of the lean epilogues moved in front of the requantisation.  With a positive multiplier
// r(a) = rne(fl(float(a) * M)) is non-decreasing in the accumulator a and r(0) = 0, so for int8 codes with zero point 0
//     clamp(sat8(r(a)), 0, six)  ==  sat8(r(clamp(a, 0, cap)))      where cap = the smallest a >= 0 with r(a) >= six,
// provided r(cap) == six (the codes do not jump over six: any multiplier below 1 qualifies).  clamp(a + bias, 0, cap) is
// ONE instruction (__viaddmin_s32_relu), against several per packed word for byte-wise max / min on the finished codes.
// Fills cap[m] per filter (INT_MAX: no upper clamp - plain ReLU, a six that saturates, or codes that never reach six) and
// returns false when some filter does not qualify (the caller then clamps the packed codes instead).
inline bool requant_relu_caps(const float* mult, size_t n, int act, int six, std::vector<int32_t>& cap) {
    cap.assign(n, 0x7fffffff);
    if (act != ZANT_QACT_RELU && act != ZANT_QACT_RELU6) return false;
    for (size_t m = 0; m < n; ++m) {
        const float M = mult[m];
        if (!(M > 0.0f) || !std::isfinite(M)) return false;
        if (act != ZANT_QACT_RELU6 || six >= 127) continue;
        auto r = [M](long long a) { return nearbyintf((float)(int)a * M); };      // the device's int -> float, multiply, rne
        if (r(0x7fffffffLL) < (float)six) continue;
        long long lo = 0, hi = 0x7fffffffLL;                                      // r(lo) < six unless six == 0; r(hi) >= six
        if (r(0) >= (float)six) hi = 0;
        while (lo < hi) { const long long mid = lo + (hi - lo) / 2; if (r(mid) >= (float)six) hi = mid; else lo = mid + 1; }
        if (r(hi) != (float)six) return false;
        cap[m] = (int32_t)hi;
    }
    return true;
}

// sat8(rne(6 / y_scale)): the code of 6.0 for int8 outputs with zero point 0 (the lean epilogues' ReLU6 bound)
inline int lean_six(float y_scale) {
    float v = 6.0f / y_scale;
    v = std::fmin(std::fmax(v, -512.0f), 511.0f);
    return std::min(std::max((int)std::nearbyintf(v), -128), 127);
}

// bytes (little endian) = sat8(a0), sat8(a1), sat8(a2), sat8(a3)
__device__ __forceinline__ uint32_t pack_sat_s8x4(int a0, int a1, int a2, int a3) {
    uint32_t hi, d;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(a3), "r"(a2));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a1), "r"(a0), "r"(hi));
    return d;
}

// bytes (little endian) = satu8(a0) .. satu8(a3), i.e. each clamped to [0, 255]
__device__ __forceinline__ uint32_t pack_sat_u8x4(int a0, int a1, int a2, int a3) {
    uint32_t hi, d;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(a3), "r"(a2));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a1), "r"(a0), "r"(hi));
    return d;
}

// Four requantised values as packed int8 codes (zero point 0) under the lean activation.  ReLU / ReLU6: the unsigned
// saturation of the pack is the lower clamp, one byte-wise unsigned minimum with `hi4` (the upper bound in every byte: the
// code of 6, or 127) the upper one - byte-wise max / min are several instructions each on this part, so one of them is
// saved against clamping signed codes from both sides.
__device__ __forceinline__ uint32_t pack_act_s8x4(int q0, int q1, int q2, int q3, bool relu, uint32_t hi4) {
    return relu ? __vminu4(pack_sat_u8x4(q0, q1, q2, q3), hi4) : pack_sat_s8x4(q0, q1, q2, q3);
}

// ReLU on four packed int8 values with zero point 0.
__device__ __forceinline__ uint32_t relu_s8x4(uint32_t v) { return __vmaxs4(v, 0u); }

template <bool U8> __device__ __forceinline__ int load_q(const void* p, size_t i) {
    return U8 ? (int)reinterpret_cast<const uint8_t*>(p)[i] : (int)reinterpret_cast<const int8_t*>(p)[i];
}
template <bool U8> __device__ __forceinline__ void store_q(void* p, size_t i, int v) {
    if (U8) reinterpret_cast<uint8_t*>(p)[i] = (uint8_t)v; else reinterpret_cast<int8_t*>(p)[i] = (int8_t)v;
}

// ---------------------------------------------------------------------------- Quantize / Dequantize
template <bool YU8>
__global__ void quantize_linear_k(const float* __restrict__ x, void* __restrict__ y, size_t n, float scale, int zp, bool vec) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    size_t done = 0;
    // sat(rne(clamp(t, -512, 511)) + zp) == rne(clamp(t, lo - zp, hi - zp)) + zp for a zero point inside the type's range:
    // the bounds are integers inside [-512, 511] and rounding is monotonic
    const bool zp_ok = YU8 ? (zp >= 0 && zp <= 255) : (zp >= -128 && zp <= 127);
    if (vec && zp_ok) {
        const QuantFast qf = quant_fast(scale, (float)((YU8 ? 0 : -128) - zp), (float)((YU8 ? 255 : 127) - zp));
        const size_t n4 = n / 4;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        uint32_t* y4 = reinterpret_cast<uint32_t*>(y);
        for (size_t i = tid; i < n4; i += stride) {
            const float4 v = x4[i];
            const int a = quantize_fast(v.x, qf) + zp;
            const int b = quantize_fast(v.y, qf) + zp;
            const int c = quantize_fast(v.z, qf) + zp;
            const int d = quantize_fast(v.w, qf) + zp;
            y4[i] = (uint32_t)(a & 255) | ((uint32_t)(b & 255) << 8) | ((uint32_t)(c & 255) << 16) | ((uint32_t)(d & 255) << 24);
        }
        done = n4 * 4;
    }
    for (size_t i = done + tid; i < n; i += stride)
        store_q<YU8>(y, i, sat_q<YU8>(rne_clamped(__fdiv_rn(x[i], scale)) + zp));
}

template <typename Q>
__global__ void dequantize_linear_k(const Q* __restrict__ q, float* __restrict__ y, size_t n, float scale, int zp) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = __fmul_rn(__int2float_rn((int)q[i] - zp), scale);
}

// ---------------------------------------------------------------------------- QLinearConv, generic
// One output per thread, ow fastest so that neighbouring threads read neighbouring inputs.
struct QConvArgs {
    const void* x; const int8_t* w; void* y;
    const float* mult;        // per-output-channel multiplier M[m] (device, length g.M)
    const int32_t* w_zp;      // per output channel (device, length g.M)
    const int32_t* bias;      // nullable
    int x_zp;
    Requant rq;
    ConvGeom g;
};

template <bool XU8, bool YU8>
__global__ void qconv_nchw_generic(const QConvArgs p) {
    const ConvGeom& g = p.g;
    const size_t total = (size_t)g.N * g.M * g.OH * g.OW;
    const int Mg = g.M / g.G;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ow = (int)(i % g.OW); size_t t = i / g.OW;
        const int oh = (int)(t % g.OH); t /= g.OH;
        const int m = (int)(t % g.M); const int n = (int)(t / g.M);
        const int grp = m / Mg;
        const int wz = p.w_zp[m];
        const int ih0 = oh * g.sh - g.pt, iw0 = ow * g.sw - g.pl;
        int acc = 0;
        for (int c = 0; c < g.Cg; ++c) {
            const size_t xplane = ((size_t)n * g.C + (size_t)grp * g.Cg + c) * g.H;
            const int8_t* wp = p.w + (((size_t)m * g.Cg + c) * g.KH) * g.KW;
            for (int kh = 0; kh < g.KH; ++kh) {
                const int ih = ih0 + kh * g.dh;
                if (ih < 0 || ih >= g.H) continue;
                for (int kw = 0; kw < g.KW; ++kw) {
                    const int iw = iw0 + kw * g.dw;
                    if (iw < 0 || iw >= g.W) continue;
                    const int xv = load_q<XU8>(p.x, (xplane + ih) * g.W + iw) - p.x_zp;
                    acc += xv * ((int)wp[kh * g.KW + kw] - wz);
                }
            }
        }
        if (p.bias) acc += p.bias[m];
        store_q<YU8>(p.y, i, requant_one<YU8>(acc, p.mult[m], p.rq));
    }
}

// ---------------------------------------------------------------------------- QLinearMatMul, generic
struct QMatArgs {
    const void* a; const int8_t* b; void* y;
    const float* mult; const int32_t* b_zp; const int32_t* bias;
    int a_zp; Requant rq;
    int M, N, K;
    int y_i32;   // store the raw accumulator
};

template <bool AU8, bool YU8>
__global__ void qmatmul_generic(const QMatArgs p) {
    const size_t total = (size_t)p.M * p.N;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(i % p.N); const size_t row = i / p.N;
        const int bz = p.b_zp[j];
        int acc = 0;
        for (int k = 0; k < p.K; ++k)
            acc += (load_q<AU8>(p.a, row * p.K + k) - p.a_zp) * ((int)p.b[(size_t)k * p.N + j] - bz);
        if (p.bias) acc += p.bias[j];
        if (p.y_i32) reinterpret_cast<int32_t*>(p.y)[i] = acc;
        else store_q<YU8>(p.y, i, requant_one<YU8>(acc, p.mult[j], p.rq));
    }
}

// ---------------------------------------------------------------------------- QLinearAdd
template <bool U8>
__global__ void qadd_k(const void* __restrict__ a, float a_s, int a_zp, const void* __restrict__ b, float b_s, int b_zp,
                       float y_s, int y_zp, int act, void* __restrict__ y, size_t n) {
    const int lo = sat_q<U8>(y_zp);
    const int six = sat_q<U8>(rne_clamped(__fdiv_rn(6.0f, y_s)) + y_zp);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float fa = __fmul_rn(__int2float_rn(load_q<U8>(a, i) - a_zp), a_s);
        const float fb = __fmul_rn(__int2float_rn(load_q<U8>(b, i) - b_zp), b_s);
        const float v = __fdiv_rn(__fadd_rn(fa, fb), y_s);
        int t = sat_q<U8>(rne_clamped(v) + y_zp);
        if (act != ZANT_QACT_NONE) t = max(t, lo);
        if (act == ZANT_QACT_RELU6) t = min(t, six);
        store_q<U8>(y, i, t);
    }
}

// The same, sixteen values per thread (16-byte loads and stores); the division by y_s goes through quantize_fast, which
// proves the rounding from a multiply and a residual and divides only where it cannot.  Requires 16-byte aligned buffers
// and a y_zp inside the type's range; the tail (n % 16 values) is left to qadd_k.
template <bool U8>
__global__ void __launch_bounds__(256) qadd_vec_k(const uint4* __restrict__ a, float a_s, int a_zp, const uint4* __restrict__ b, float b_s, int b_zp,
                                                  float y_s, int y_zp, int act, uint4* __restrict__ y, size_t n16) {
    const int t_lo = U8 ? 0 : -128, t_hi = U8 ? 255 : 127;
    const QuantFast qf = quant_fast(y_s, (float)(t_lo - y_zp), (float)(t_hi - y_zp));
    const int lo = sat_q<U8>(y_zp);
    const int six = sat_q<U8>(rne_clamped(__fdiv_rn(6.0f, y_s)) + y_zp);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 va = __ldg(a + i), vb = __ldg(b + i);
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint32_t out[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t pk = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int qa = U8 ? (int)((wa[w] >> (8 * j)) & 255u) : (int)(int8_t)(wa[w] >> (8 * j));
                const int qb = U8 ? (int)((wb[w] >> (8 * j)) & 255u) : (int)(int8_t)(wb[w] >> (8 * j));
                const float fa = __fmul_rn(__int2float_rn(qa - a_zp), a_s);
                const float fb = __fmul_rn(__int2float_rn(qb - b_zp), b_s);
                int t = quantize_fast(__fadd_rn(fa, fb), qf) + y_zp;
                if (act != ZANT_QACT_NONE) t = max(t, lo);
                if (act == ZANT_QACT_RELU6) t = min(t, six);
                pk |= (uint32_t)(t & 255) << (8 * j);
            }
            out[w] = pk;
        }
        y[i] = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// ---------------------------------------------------------------------------- Quantized GlobalAveragePool
// One warp per (n,c) plane: exact int32 sum by shuffle reduction (integer addition is
// associative, so the order is free), then the three rounded fp32 steps.
template <bool U8>
__global__ void qgap_k(const void* __restrict__ x, void* __restrict__ y, size_t planes, int hw,
                       float x_s, int x_zp, float y_s, int y_zp) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t pidx = warp; pidx < planes; pidx += nwarps) {
        int s = 0;
        for (int j = lane; j < hw; j += 32) s += load_q<U8>(x, pidx * hw + j) - x_zp;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            const float f = __fmul_rn(__int2float_rn(s), x_s);
            const float mean = __fdiv_rn(f, (float)hw);
            const float v = __fdiv_rn(mean, y_s);
            store_q<U8>(y, pidx, sat_q<U8>(rne_clamped(v) + y_zp));
        }
    }
}

// Small planes (a few dozen bytes, as behind the last stage of a mobile network): one THREAD per plane.  The plane's bytes are
// summed four at a time (dp4a against ones) from the aligned words that hold them, the bytes of the neighbouring planes
// masked out of the first and last word; neighbouring threads read neighbouring runs, so every fetched line is used in full.
// x must be 4-byte aligned; the word that holds the tensor's last bytes is read byte by byte when it is not whole.
template <bool U8>
__global__ void qgap_small_k(const uint8_t* __restrict__ x, void* __restrict__ y, size_t planes, int hw,
                             float x_s, int x_zp, float y_s, int y_zp) {
    const size_t total = planes * (size_t)hw;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t pidx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; pidx < planes; pidx += stride) {
        const size_t a = pidx * hw, b = a + hw;                  // the plane's bytes [a, b)
        int s = 0;
        for (size_t w = a >> 2; w * 4 < b; ++w) {
            uint32_t v;
            if (w * 4 + 4 <= total) v = __ldg(reinterpret_cast<const uint32_t*>(x) + w);
            else { v = 0; for (size_t i = w * 4; i < total; ++i) v |= (uint32_t)__ldg(x + i) << (8 * (i & 3)); }
            uint32_t keep = 0xffffffffu;
            if (w * 4 < a) keep &= 0xffffffffu << (8 * (uint32_t)(a - w * 4));
            if (w * 4 + 4 > b) keep &= 0xffffffffu >> (8 * (uint32_t)(w * 4 + 4 - b));
            v &= keep;
            if (U8) asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(s) : "r"(v), "r"(0x01010101u), "r"(s));
            else asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(s) : "r"(v), "r"(0x01010101u), "r"(s));
        }
        s -= hw * x_zp;
        const float f = __fmul_rn(__int2float_rn(s), x_s);
        const float mean = __fdiv_rn(f, (float)hw);
        const float v = __fdiv_rn(mean, y_s);
        store_q<U8>(y, pidx, sat_q<U8>(rne_clamped(v) + y_zp));
    }
}

// ---------------------------------------------------------------------------- 256-entry table lookup
__global__ void lut_q8_k(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, size_t n, const uint8_t* __restrict__ lut_g, bool vec) {
    __shared__ uint8_t lut[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = lut_g[i];
    __syncthreads();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    size_t done = 0;
    if (vec) {
        const size_t n16 = n / 16;
        const uint4* x4 = reinterpret_cast<const uint4*>(x);
        uint4* y4 = reinterpret_cast<uint4*>(y);
        for (size_t i = tid; i < n16; i += stride) {
            uint4 v = x4[i];
            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t u = w[k];
                w[k] = (uint32_t)lut[u & 255] | ((uint32_t)lut[(u >> 8) & 255] << 8) |
                       ((uint32_t)lut[(u >> 16) & 255] << 16) | ((uint32_t)lut[u >> 24] << 24);
            }
            y4[i] = v;
        }
        done = n16 * 16;
    }
    for (size_t i = done + tid; i < n; i += stride) y[i] = lut[x[i]];
}

}  // namespace zb
