// FP32 kernels with the reference's arithmetic: every dot product is accumulated by ONE
// thread in ascending k with a separate multiply and add (__fmul_rn/__fadd_rn are never
// contracted into an FMA), so results are bit-identical to the reference's CPU loops.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "geometry.hpp"

namespace zb {

// ------------------------------------------------------------------------------------------
// Tiled contraction  D[m,j] = sum_k A(m,k) * B(k,j)
//   CONV = true : A is gathered on the fly from an NCHW input (implicit im2col, k = (c,kh,kw)
//                 exactly as lean_im2col orders it), B(k,j) = W[j*K + k], D scattered to NCHW
//                 with the bias added after the sum (op_convolution.zig:316-328).
//   CONV = false: A(m,k) = a[m*sam + k*sak], B(k,j) = b[k*sbk + j*sbj] (covers MatMul and the
//                 transposed operands of Gemm), then  v*alpha  and  + c*beta  as two separately
//                 rounded steps (op_gemm.zig:128-178).
// 64x64 output tile per CTA, 16-wide k slabs in shared memory, 4x4 outputs per thread.
// ------------------------------------------------------------------------------------------
struct ContractArgs {
    const float* a; const float* b; float* d;
    int M, N, K;
    // plain-matrix strides (elements)
    long long sam, sak, sbk, sbj;
    // conv gather
    ConvGeom g;
    const float* bias;
    // gemm epilogue
    int epilogue;            // 0 plain store, 1 gemm (alpha, optional C)
    float alpha, beta;
    const float* c; int c_mode; long long c_rs, c_cs;   // c index = m*c_rs + j*c_cs
};

constexpr int CT_BM = 64, CT_BN = 64, CT_BK = 16, CT_PAD = 4;

template <bool CONV>
__global__ void __launch_bounds__(256) contract_f32_exact(const ContractArgs p) {
    __shared__ float As[CT_BK][CT_BM + CT_PAD];
    __shared__ float Bs[CT_BK][CT_BN + CT_PAD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4x4 outputs each
    const int m0 = blockIdx.x * CT_BM, j0 = blockIdx.y * CT_BN;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // ---- A loader mapping
    // conv / column-contiguous A: consecutive threads walk m (coalesced along ow);
    // row-contiguous A (sak == 1): consecutive threads walk k.
    const bool a_kfast = !CONV && p.sak == 1;
    const int a_m = a_kfast ? (tid >> 4) : (tid & 63);     // + 16*i (k-fast)  |  fixed (m-fast)
    const int a_k = a_kfast ? (tid & 15) : (tid >> 6);     // fixed (k-fast)    |  + 4*i (m-fast)
    // conv: decode this thread's row once
    int cn = 0, ih0 = 0, iw0 = 0;
    bool row_ok = false;
    if (CONV) {
        const int m = m0 + a_m;
        row_ok = m < p.M;
        if (row_ok) {
            const int ow = m % p.g.OW; const int t = m / p.g.OW;
            const int oh = t % p.g.OH; cn = t / p.g.OH;
            ih0 = oh * p.g.sh - p.g.pt; iw0 = ow * p.g.sw - p.g.pl;
        }
    }
    const int khw = p.g.KH * p.g.KW;
    // ---- B loader mapping: k-fast when B is k-contiguous (conv weights), else j-fast
    const bool b_kfast = CONV || p.sbk == 1;
    const int b_j = b_kfast ? (tid >> 4) : (tid & 63);
    const int b_k = b_kfast ? (tid & 15) : (tid >> 6);

    for (int k0 = 0; k0 < p.K; k0 += CT_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v = 0.0f;
            if (CONV) {
                const int k = k0 + a_k + 4 * i;
                if (row_ok && k < p.K) {
                    const int c = k / khw; const int r = k - c * khw;
                    const int kh = r / p.g.KW; const int kw = r - kh * p.g.KW;
                    const int ih = ih0 + kh * p.g.dh, iw = iw0 + kw * p.g.dw;
                    if (ih >= 0 && ih < p.g.H && iw >= 0 && iw < p.g.W)
                        v = __ldg(p.a + (((long long)cn * p.g.C + c) * p.g.H + ih) * p.g.W + iw);
                }
                As[a_k + 4 * i][a_m] = v;
            } else if (a_kfast) {
                const int m = m0 + a_m + 16 * i, k = k0 + a_k;
                if (m < p.M && k < p.K) v = __ldg(p.a + (long long)m * p.sam + (long long)k * p.sak);
                As[a_k][a_m + 16 * i] = v;
            } else {
                const int m = m0 + a_m, k = k0 + a_k + 4 * i;
                if (m < p.M && k < p.K) v = __ldg(p.a + (long long)m * p.sam + (long long)k * p.sak);
                As[a_k + 4 * i][a_m] = v;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v = 0.0f;
            if (b_kfast) {
                const int j = j0 + b_j + 16 * i, k = k0 + b_k;
                if (j < p.N && k < p.K)
                    v = CONV ? __ldg(p.b + (long long)j * p.K + k)
                             : __ldg(p.b + (long long)k * p.sbk + (long long)j * p.sbj);
                Bs[b_k][b_j + 16 * i] = v;
            } else {
                const int j = j0 + b_j, k = k0 + b_k + 4 * i;
                if (j < p.N && k < p.K) v = __ldg(p.b + (long long)k * p.sbk + (long long)j * p.sbj);
                Bs[b_k + 4 * i][b_j] = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < CT_BK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
        if (CONV) {
            const int ow = m % p.g.OW; const int t = m / p.g.OW;
            const int oh = t % p.g.OH; const int n = t / p.g.OH;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int f = j0 + tx * 4 + j;
                if (f >= p.N) continue;
                const float bv = p.bias ? __ldg(p.bias + f) : 0.0f;
                p.d[(((long long)n * p.g.M + f) * p.g.OH + oh) * p.g.OW + ow] = __fadd_rn(acc[i][j], bv);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = j0 + tx * 4 + j;
                if (col >= p.N) continue;
                float v = acc[i][j];
                if (p.epilogue == 1) {
                    v = __fmul_rn(v, p.alpha);
                    if (p.c_mode) v = __fadd_rn(v, __fmul_rn(__ldg(p.c + (long long)m * p.c_rs + (long long)col * p.c_cs), p.beta));
                }
                p.d[(long long)m * p.N + col] = v;
            }
        }
    }
}

// Element-wise pass over the part of a Gemm result that lies beyond the first matrix of a
// batched tensor: the reference scales the WHOLE result tensor by alpha and adds beta*C to all
// of it (op_gemm.zig:130-178) although only the first [rows x cols] block holds a product.
__global__ void gemm_tail_f32(float* y, size_t begin, size_t total, float alpha,
                              const float* c, int c_mode, float beta,
                              size_t rows, size_t cols, size_t c_rows, size_t c_cols, size_t y_ch, size_t c_ch) {
    for (size_t i = begin + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = __fmul_rn(0.0f, alpha);   // untouched elements hold the zero the caller cleared them to
        (void)y_ch;
        if (c_mode == 1) v = __fadd_rn(v, __fmul_rn(c[i], beta));
        else if (c_mode == 2) {
            const size_t col = i % cols; size_t t = i / cols;
            const size_t row = t % rows; t /= rows;          // t = b*y_ch + ch
            const size_t ci = c_rows == 1 ? 0 : row, cj = c_cols == 1 ? 0 : col;
            v = __fadd_rn(v, __fmul_rn(c[(t * c_rows + ci) * c_cols + cj], beta));
        }
        (void)c_ch;
        y[i] = v;
    }
}

// ------------------------------------------------------------------------------------------
// MaxPool (lean_onnx_maxpool, op_pooling.zig:620-658) — one output per thread, NCHW planes.
// T = float (init -inf), int8_t (-128) or uint8_t (0).
// ------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ T pool_init();
template <> __device__ __forceinline__ float pool_init<float>() { return -INFINITY; }
template <> __device__ __forceinline__ int8_t pool_init<int8_t>() { return -128; }
template <> __device__ __forceinline__ uint8_t pool_init<uint8_t>() { return 0; }

template <typename T>
__global__ void maxpool_nchw(const T* __restrict__ x, T* __restrict__ y, const PoolGeom g) {
    const size_t total = (size_t)g.NC * g.OH * g.OW;
    const bool small = total < 0xffffffffull;         // 32-bit index arithmetic: 64-bit division costs hundreds of instructions
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int ow, oh; size_t plane;
        if (small) {
            const uint32_t i32 = (uint32_t)i, t = i32 / (uint32_t)g.OW, pl = t / (uint32_t)g.OH;
            ow = (int)(i32 - t * (uint32_t)g.OW); oh = (int)(t - pl * (uint32_t)g.OH); plane = pl;
        } else {
            ow = (int)(i % g.OW); const size_t t = i / g.OW;
            oh = (int)(t % g.OH); plane = t / g.OH;
        }
        const T* xp = x + plane * (size_t)g.H * g.W;
        const int ih0 = oh * g.sh - g.pt, iw0 = ow * g.sw - g.pl;
        T m = pool_init<T>();
        for (int kh = 0; kh < g.KH; ++kh) {
            const int ih = ih0 + kh * g.dh;
            if (ih < 0 || ih >= g.H) continue;
            for (int kw = 0; kw < g.KW; ++kw) {
                const int iw = iw0 + kw * g.dw;
                if (iw < 0 || iw >= g.W) continue;
                const T v = xp[(size_t)ih * g.W + iw];
                m = v > m ? v : m;
            }
        }
        y[i] = m;
    }
}

// 2x2 / stride 2 / no padding on 8-bit planes whose rows are whole 8-byte groups (W % 8 == 0, even H):
// a thread reads 8 bytes of two input rows, takes the row-wise maximum with one packed byte-max, then
// the maximum of neighbouring bytes, and stores 4 outputs.  Same values as maxpool_nchw.
template <bool SIGNED>
__global__ void maxpool2x2s2_q8(const uint2* __restrict__ x, uint32_t* __restrict__ y, size_t planes_rows, int ow4, int w8) {
    // planes_rows = NC * OH output rows; an output row has ow4 words, its two input rows have w8 (= ow4) uint2 each
    const size_t total = planes_rows * (size_t)ow4;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / ow4;
        const int c = (int)(i - row * ow4);
        const uint2 a = __ldg(x + (row * 2) * (size_t)w8 + c), b = __ldg(x + (row * 2 + 1) * (size_t)w8 + c);
        const uint32_t m0 = SIGNED ? __vmaxs4(a.x, b.x) : __vmaxu4(a.x, b.x);
        const uint32_t m1 = SIGNED ? __vmaxs4(a.y, b.y) : __vmaxu4(a.y, b.y);
        const uint32_t even = __byte_perm(m0, m1, 0x6420), odd = __byte_perm(m0, m1, 0x7531);
        y[i] = SIGNED ? __vmaxs4(even, odd) : __vmaxu4(even, odd);
    }
}

// The float form: a thread reads a float4 of two input rows and stores two outputs.  The maximum is taken with the
// reference's comparison chain (start at -inf, take a value only if it is greater), in the window's kh, kw order, so NaNs
// are skipped exactly as there.
__global__ void maxpool2x2s2_f32(const float4* __restrict__ x, float2* __restrict__ y, size_t planes_rows, int ow2, int w4) {
    const size_t total = planes_rows * (size_t)ow2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / ow2;
        const int c = (int)(i - row * ow2);
        const float4 a = __ldg(x + (row * 2) * (size_t)w4 + c), b = __ldg(x + (row * 2 + 1) * (size_t)w4 + c);
        float m0 = -INFINITY, m1 = -INFINITY;
        m0 = a.x > m0 ? a.x : m0; m0 = a.y > m0 ? a.y : m0; m0 = b.x > m0 ? b.x : m0; m0 = b.y > m0 ? b.y : m0;
        m1 = a.z > m1 ? a.z : m1; m1 = a.w > m1 ? a.w : m1; m1 = b.z > m1 ? b.z : m1; m1 = b.w > m1 ? b.w : m1;
        y[i] = make_float2(m0, m1);
    }
}

// ------------------------------------------------------------------------------------------
// Element-wise activations: float4 body when both pointers are 16-byte aligned, scalar tail.
// ------------------------------------------------------------------------------------------
struct ReluOp { __device__ float operator()(float v) const { return v > 0.0f ? v : 0.0f; } };
struct LeakyOp { float slope; __device__ float operator()(float v) const { return v <= 0.0f ? __fmul_rn(slope, v) : v; } };
struct ClipOp { float lo, hi; __device__ float operator()(float v) const { return fminf(fmaxf(v, lo), hi); } };
// sigmoid_lean, tanh_lean, ceil_lean: exp / tanh are the CUDA library's accurate single-precision forms
// (they agree with the reference's within a few units in the last place, inside the FP32 tolerance).
struct SigmoidOp { __device__ float operator()(float v) const { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))); } };
struct TanhOp { __device__ float operator()(float v) const { return tanhf(v); } };
struct CeilOp { __device__ float operator()(float v) const { return (isnan(v) || isinf(v)) ? v : ceilf(v); } };

// mul_lean / div_lean: equal sizes, one rounded operation per element.
template <bool DIV>
__global__ void binary_same_f32(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = DIV ? __fdiv_rn(a[i], b[i]) : __fmul_rn(a[i], b[i]);
}

// lean_softmax: one thread per row walks it three times in index order (maximum; exp and running sum;
// division), which reproduces the reference's summation order.
__global__ void softmax_rows_f32(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols) {
    for (size_t r = blockIdx.x * (size_t)blockDim.x + threadIdx.x; r < rows; r += (size_t)gridDim.x * blockDim.x) {
        if (cols == 0) continue;
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float m = xr[0];
        for (size_t j = 0; j < cols; ++j) m = xr[j] > m ? xr[j] : m;
        float sum = 0.0f;
        for (size_t j = 0; j < cols; ++j) { const float v = expf(__fsub_rn(xr[j], m)); yr[j] = v; sum = __fadd_rn(sum, v); }
        for (size_t j = 0; j < cols; ++j) yr[j] = __fdiv_rn(yr[j], sum);
    }
}

template <typename F>
__global__ void unary_f32(const float* __restrict__ x, float* __restrict__ y, size_t n, bool vec, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    size_t done = 0;
    if (vec) {
        const size_t n4 = n / 4;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        float4* y4 = reinterpret_cast<float4*>(y);
        for (size_t i = tid; i < n4; i += stride) {
            float4 v = x4[i];
            v.x = f(v.x); v.y = f(v.y); v.z = f(v.z); v.w = f(v.w);
            y4[i] = v;
        }
        done = n4 * 4;
    }
    for (size_t i = done + tid; i < n; i += stride) y[i] = f(x[i]);
}

// Add of equal-sized tensors (lib_elementWise_math.zig:72-110).
__global__ void add_same_f32(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, size_t n, bool vec) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    size_t done = 0;
    if (vec) {
        const size_t n4 = n / 4;
        const float4* a4 = reinterpret_cast<const float4*>(a);
        const float4* b4 = reinterpret_cast<const float4*>(b);
        float4* y4 = reinterpret_cast<float4*>(y);
        for (size_t i = tid; i < n4; i += stride) {
            const float4 u = a4[i], v = b4[i];
            y4[i] = make_float4(__fadd_rn(u.x, v.x), __fadd_rn(u.y, v.y), __fadd_rn(u.z, v.z), __fadd_rn(u.w, v.w));
        }
        done = n4 * 4;
    }
    for (size_t i = done + tid; i < n; i += stride) y[i] = __fadd_rn(a[i], b[i]);
}

// Broadcasting Add up to rank 4 (lib_elementWise_math.zig:112-209).
struct BcastArgs { int rank; size_t out_shape[4]; size_t a_stride[4]; size_t b_stride[4]; size_t total; };
__global__ void add_bcast_f32(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, const BcastArgs g) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < g.total; i += (size_t)gridDim.x * blockDim.x) {
        size_t rem = i, ia = 0, ib = 0;
        for (int d = g.rank - 1; d >= 0; --d) {
            const size_t pos = rem % g.out_shape[d];
            rem /= g.out_shape[d];
            ia += pos * g.a_stride[d]; ib += pos * g.b_stride[d];
        }
        y[i] = __fadd_rn(a[ia], b[ib]);
    }
}

// Sum of a tensor list in list order (lib_elementWise_math.zig:243-257).
struct SumListArgs { const float* t[8]; int n; };
__global__ void sum_list_f32(const SumListArgs l, float* __restrict__ y, size_t n, bool accumulate) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float s = accumulate ? y[i] : l.t[0][i];
        for (int k = accumulate ? 0 : 1; k < l.n; ++k) s = __fadd_rn(s, l.t[k][i]);
        y[i] = s;
    }
}

// ------------------------------------------------------------------------------------------
// Strided 2-D byte copy: rows of `row_bytes` from src (pitch sp) to dst (pitch dp).  Used by
// Concat (one launch per input tensor).  Word = uint4 / uint32_t / uint8_t by alignment.
// ------------------------------------------------------------------------------------------
template <typename Word>
__global__ void copy2d(const char* __restrict__ src, size_t sp, char* __restrict__ dst, size_t dp,
                       size_t row_words, size_t rows) {
    const size_t total = row_words * rows;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / row_words, w = i - r * row_words;
        reinterpret_cast<Word*>(dst + r * dp)[w] = reinterpret_cast<const Word*>(src + r * sp)[w];
    }
}

// ------------------------------------------------------------------------------------------
// Resize nearest: out[o] = in[sum_d table_d[o_d] * istride_d]; the per-axis source-index
// tables are computed on the host with the reference's fp32 formula.
// ------------------------------------------------------------------------------------------
struct ResizeArgs { int rank; size_t out_shape[8]; size_t in_stride[8]; int axis_offset[8]; size_t total; };
// IDX: the type of the index arithmetic - 32 bits when both tensors have fewer than 2^31 elements (64-bit division and
// modulo cost hundreds of instructions per element; with them a 2.8 M-element nearest-neighbour upsampling took 33 us).
template <typename T, typename IDX>
__global__ void resize_gather(const T* __restrict__ x, T* __restrict__ y, const int32_t* __restrict__ table, const ResizeArgs g) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < g.total; i += (size_t)gridDim.x * blockDim.x) {
        IDX rem = (IDX)i, src = 0;
        for (int d = g.rank - 1; d >= 0; --d) {
            const IDX n = (IDX)g.out_shape[d];
            const IDX q = rem / n, pos = rem - q * n;
            rem = q;
            src += (IDX)table[g.axis_offset[d] + pos] * (IDX)g.in_stride[d];
        }
        y[i] = x[src];
    }
}

// ------------------------------------------------------------------------------------------
// ReduceMean: one output per thread, reduced coordinates visited in the reference's order
// (last listed axis fastest), sequential fp32 sum, one division (lib_reduction_math.zig:226-266).
// ------------------------------------------------------------------------------------------
struct ReduceArgs {
    size_t out_total, count; int n_keep, n_red;
    size_t keep_ostride[8], keep_istride[8], red_size[8], red_istride[8];
};
__global__ void reduce_mean_f32(const float* __restrict__ x, float* __restrict__ y, const ReduceArgs g) {
    for (size_t o = blockIdx.x * (size_t)blockDim.x + threadIdx.x; o < g.out_total; o += (size_t)gridDim.x * blockDim.x) {
        size_t rem = o, base = 0;
        for (int i = 0; i < g.n_keep; ++i) { base += (rem / g.keep_ostride[i]) * g.keep_istride[i]; rem %= g.keep_ostride[i]; }
        float s = 0.0f;
        if (g.n_red == 2) {
            for (size_t i1 = 0; i1 < g.red_size[1]; ++i1)
                for (size_t i0 = 0; i0 < g.red_size[0]; ++i0)
                    s = __fadd_rn(s, x[base + i1 * g.red_istride[1] + i0 * g.red_istride[0]]);
        } else {
            for (size_t idx = 0; idx < g.count; ++idx) {
                size_t t = idx, off = base;
                for (int d = 0; d < g.n_red; ++d) { off += (t % g.red_size[d]) * g.red_istride[d]; t /= g.red_size[d]; }
                s = __fadd_rn(s, x[off]);
            }
        }
        y[o] = __fdiv_rn(s, (float)g.count);
    }
}

// Mean of ALL elements into y[0] with the reference's strictly sequential sum
// (lib_reduction_math.zig:120-128).  One thread: the order of additions is the contract.
__global__ void reduce_all_mean_f32(const float* __restrict__ x, float* __restrict__ y, size_t n) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        float s = 0.0f;
        for (size_t i = 0; i < n; ++i) s = __fadd_rn(s, x[i]);
        y[0] = __fdiv_rn(s, (float)n);
    }
}

// ------------------------------------------------------------------------------------------
// Transpose / Slice: y[i] = x[base + sum_d coord_d(i) * in_stride[d]], coordinates of the row-major
// output index.  Gather: y[(o * n_idx + k) * inner + j] = x[(o * axis_dim + idx[k]) * inner + j].
// T is an unsigned type of the element's size.
// ------------------------------------------------------------------------------------------
struct StridedMapDev { int rank; long long out_dims[8]; long long in_stride[8]; long long base; size_t total; };

template <typename T>
__global__ void strided_copy_k(const T* __restrict__ x, T* __restrict__ y, const StridedMapDev m) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < m.total; i += (size_t)gridDim.x * blockDim.x) {
        size_t t = i;
        long long src = m.base;
        for (int d = m.rank - 1; d >= 0; --d) {
            const size_t c = t % (size_t)m.out_dims[d];
            t /= (size_t)m.out_dims[d];
            src += (long long)c * m.in_stride[d];
        }
        y[i] = x[src];
    }
}

template <typename T>
__global__ void gather_axis_k(const T* __restrict__ x, const int32_t* __restrict__ idx, T* __restrict__ y,
                              size_t outer, size_t n_idx, size_t inner, size_t axis_dim) {
    const size_t total = outer * n_idx * inner;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t j = i % inner, t = i / inner;
        const size_t k = t % n_idx, o = t / n_idx;
        y[i] = x[(o * axis_dim + (size_t)idx[k]) * inner + j];
    }
}

}  // namespace zb
