// Float contractions on the tensor cores: tcgen05.mma kind::tf32 with fp32 accumulation in TMEM.
//
// This is the 2e-3 path of the float operators (Conv, MatMul, Gemm), selected per context
// (zant_b200_ctx_set_tf32); the default stays the exact FP32 kernels, which keep the reference's
// order of operations.  A convolution is an im2col gather into the GEMM-blocked operand layout
// followed by the GEMM; a matrix product blocks its left operand the same way.
//
// Operand layout (the byte geometry of the int8 GEMM, with 4-byte elements): rows are grouped in
// tiles (128 rows of A, NT rows of W^T), K is split into 16-byte chunks of four floats, chunk-major:
//   [tile][K/4][rows][4] float
// so that a run of chunks of one tile is one bulk async copy and lands in shared memory as the K-major,
// no-swizzle operand of an MMA whose K step is 8 floats = 32 bytes = two chunks.  Operands are rounded to
// TF32 (nearest, ties away) when they are blocked - the gather does it for A, the host for the weights -
// because the tensor core would otherwise truncate them, which biases long sums.
//
// Two precisions.  Single pass: one MMA per K step on the rounded operands; the error of a sum is about
// 3e-4 * sqrt(sum of squared products), i.e. small against the output's scale but not against an output that is
// itself a near-cancellation.  Split ("3 x TF32"): every operand is carried as hi = tf32(v) and lo = tf32(v - hi),
// and a K step issues A_hi*W_hi + A_lo*W_hi + A_hi*W_lo, which recovers about 21 bits of the products; a pipeline stage
// then holds [hi chunks][lo chunks] of both operands.
//
// Persistent CTAs, one per SM; warp roles as in the int8 GEMM:
//   warp 0    producer (bulk copies, STAGES-deep mbarrier ring)     warp 1   TMEM owner + MMA issuer
//   warps 2-9 epilogue: TMEM -> registers, + bias, ReLU / LeakyReLU, store (row-major or NCHW)
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <vector>

#include "context.cuh"
#include "fused_cnn.cuh"
#include "geometry.hpp"
#include "ptx_sm100.cuh"

namespace zb {

enum FAct { FACT_NONE = 0, FACT_RELU = 1, FACT_LEAKY = 2 };

struct TfGemmArgs {
    const float* a;        // [ceil(M/128)][K4/KC stages][parts][KC][128][4]   (parts: hi, and lo in the split form)
    const float* w;        // [N/NT][K4/KC stages][parts][KC][NT][4]
    const float* bias;     // [N] (zeros when the operator has none)
    float* y;
    int M, N, K4;          // N = padded column count (multiple of NT), K4 = chunks of four floats, a multiple of KC
    int n_valid;           // real columns
    int ohw;               // > 0: rows are (image, position) and the result is stored NCHW with ohw positions per image; 0: row-major [M][n_valid]
    int act; float slope;  // FAct
    int* status;
};

// Instruction descriptor for kind::tf32: fp32 accumulator, TF32 A and B, both K-major.
__host__ __device__ constexpr uint32_t idesc_tf32(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    const uint32_t zero = 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc), "r"(zero) : "memory");
}

__device__ __forceinline__ float round_tf32(float v) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    return __uint_as_float(u);
}

template <int NT, int KC, int STAGES, bool SPLIT = false>
struct TfGemmCfg {
    static constexpr int PARTS = SPLIT ? 2 : 1;
    static constexpr int A_PART = KC * 128 * 16;
    static constexpr int W_PART = KC * NT * 16;
    static constexpr int A_STAGE = PARTS * A_PART;
    static constexpr int W_STAGE = PARTS * W_PART;
    static constexpr int STAGE = A_STAGE + W_STAGE;
    static constexpr int MAX_N = 2048;                       // bias kept in shared memory
    static constexpr int OFF_CONST = STAGES * STAGE;
    static constexpr int OFF_BAR = OFF_CONST + MAX_N * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 512;
    static constexpr int TMEM_COLS = 2 * NT;
    static constexpr int THREADS = 320;
    static constexpr int COLS_PER_WARP = NT / 2;
    static_assert(KC % 2 == 0 && NT % 64 == 0 && NT <= 256, "tile shape");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

template <int NT, int KC, int STAGES, bool SPLIT>
__global__ void __launch_bounds__(320, 1) tc_gemm_tf32_kernel(const __grid_constant__ TfGemmArgs a) {
    using Cfg = TfGemmCfg<NT, KC, STAGES, SPLIT>;
    extern __shared__ __align__(1024) uint8_t smem[];
    float* sBias = reinterpret_cast<float*>(smem + Cfg::OFF_CONST);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 400);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 404);
    volatile int* epi_ok = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 408);
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = a.N / NT;
    const int m_tiles = (a.M + 127) / 128;
    const int tiles = m_tiles * n_tiles;
    const int k_stages = a.K4 / KC;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(full(s), 1); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), 8); }
        *abort_flag = 0;
        *epi_ok = 1;
        ptx::mbar_fence_init();
    }
    for (int i = tid; i < a.N; i += Cfg::THREADS) sBias[i] = __ldg(a.bias + i);
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (ptx::elect_one()) {
            int it = 0;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
                const int m = t / n_tiles, n = t - m * n_tiles;
                const uint8_t* ga = reinterpret_cast<const uint8_t*>(a.a) + (size_t)m * a.K4 * (Cfg::PARTS * 2048);
                const uint8_t* gw = reinterpret_cast<const uint8_t*>(a.w) + (size_t)n * a.K4 * (Cfg::PARTS * NT * 16);
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) goto producer_done;
                    ptx::mbar_arrive_expect_tx(full(s), Cfg::STAGE);
                    const uint32_t dst = ptx::smem_u32(smem + s * Cfg::STAGE);
                    ptx::bulk_g2s(dst, ga + (size_t)ks * Cfg::A_STAGE, Cfg::A_STAGE, full(s));
                    ptx::bulk_g2s(dst + Cfg::A_STAGE, gw + (size_t)ks * Cfg::W_STAGE, Cfg::W_STAGE, full(s));
                }
            }
        producer_done:;
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = idesc_tf32(128, NT);
            int it = 0, tile_it = 0;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
                const int b = tile_it & 1;
                const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
                if (!ptx::mbar_wait(tempty(b), bph ^ 1u, abort_flag)) goto mma_done;
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * NT);
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!ptx::mbar_wait(full(s), ph, abort_flag)) goto mma_done;
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + s * Cfg::STAGE);
                    const uint32_t sw = sa + Cfg::A_STAGE;
#pragma unroll
                    for (int kk = 0; kk < KC / 2; ++kk) {
                        const uint64_t da = ptx::smem_desc_kmajor(sa + (uint32_t)(kk * 2 * 2048), 2048, 128);
                        const uint64_t db = ptx::smem_desc_kmajor(sw + (uint32_t)(kk * 2 * NT * 16), NT * 16, 128);
                        if constexpr (SPLIT) {
                            // the two correction terms first, the leading term last
                            const uint64_t da_lo = ptx::smem_desc_kmajor(sa + (uint32_t)(Cfg::A_PART + kk * 2 * 2048), 2048, 128);
                            const uint64_t db_lo = ptx::smem_desc_kmajor(sw + (uint32_t)(Cfg::W_PART + kk * 2 * NT * 16), NT * 16, 128);
                            mma_tf32(d_tmem, da_lo, db, idesc, (ks | kk) != 0);
                            mma_tf32(d_tmem, da, db_lo, idesc, true);
                            mma_tf32(d_tmem, da, db, idesc, true);
                        } else {
                            mma_tf32(d_tmem, da, db, idesc, (ks | kk) != 0);
                        }
                    }
                    ptx::mma_commit(empty(s));
                }
                ptx::mma_commit(tfull(b));
            }
        mma_done:;
        }
    } else {
        // epilogue: warp (2+q) and (6+q) read lane quarter q; the first four warps take the tile's left half of the columns
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        const int e = (warp - 2) * 32 + lane;
        int tile_it = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
            const int m = t / n_tiles, n = t - m * n_tiles;
            const int b = tile_it & 1;
            const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
            if (e == 0) *epi_ok = ptx::mbar_wait(tfull(b), bph, abort_flag) ? 1 : 0;
            ptx::named_barrier_sync(1, 256);
            if (!*epi_ok) break;
            ptx::tc_fence_after();
            const int tcol0 = half * Cfg::COLS_PER_WARP;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * NT + tcol0);
            const int grow = m * 128 + row;
            const bool row_ok = grow < a.M;
            float* ybase;
            size_t col_stride;
            if (a.ohw > 0) {           // NCHW: for a fixed channel a warp writes 32 consecutive floats
                const int img = grow / a.ohw, pos = grow - img * a.ohw;
                ybase = a.y + (size_t)img * a.n_valid * a.ohw + pos;
                col_stride = (size_t)a.ohw;
            } else {
                ybase = a.y + (size_t)grow * a.n_valid;
                col_stride = 1;
            }
#pragma unroll 1
            for (int h = 0; h < Cfg::COLS_PER_WARP / 16; ++h) {
                const int col0 = n * NT + tcol0 + h * 16;
                if (col0 >= a.n_valid) break;                      // column padding of the last tile: nothing to compute or store
                uint32_t v[16];
                ptx::tmem_ld16(taddr + (uint32_t)(h * 16), v);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float r = __fadd_rn(__uint_as_float(v[j]), sBias[col0 + j]);
                    if (a.act == FACT_RELU) r = r > 0.0f ? r : 0.0f;
                    else if (a.act == FACT_LEAKY) r = r <= 0.0f ? __fmul_rn(a.slope, r) : r;
                    v[j] = __float_as_uint(r);
                }
                if (!row_ok) continue;
                if (a.ohw == 0 && (a.n_valid & 3) == 0 && col0 + 16 <= a.n_valid) {
                    // row-major: the lane's 16 columns are contiguous (rows start at multiples of 16 bytes)
                    uint4* dst = reinterpret_cast<uint4*>(ybase + col0);
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) dst[j4] = make_uint4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (col0 + j < a.n_valid) ybase[(size_t)(col0 + j) * col_stride] = __uint_as_float(v[j]);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty(b));
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    if (tid == 0 && *abort_flag) atomicExch(a.status, (int)DEV_ERR_WAIT_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// Operand blocking
// ---------------------------------------------------------------------------------------------
struct TfIm2colArgs {
    const float* x; float* a;
    ConvGeom g;
    long long rows;        // N * OH * OW
    int K, K4;             // K = Cg * KH * KW (reference order c, kh, kw); K4 chunks including padding
    int KC, parts;         // chunks per pipeline stage; 1 = rounded operand only, 2 = hi and lo parts
    const int2* ktab;      // [K4 * 4]: x = element offset of tap k from the patch origin (c*H*W + kh*dh*W + kw*dw),
                           //           y = kh*dh | kw*dw << 16, or -1 for the K padding
};

// Where chunk `kc` (part `part`) of row `r` of row tile `tile` lives, in float4 units: [tile][stage][part][KC][128]
// (KC is 4 or 8: shifts instead of divisions)
__device__ __forceinline__ long long tf_chunk_index(long long tile, int kc, int part, int r, int K4, int KC, int parts) {
    const int sh = KC == 8 ? 3 : 2;
    const int stage = kc >> sh, j = kc & (KC - 1);
    return (((tile * (K4 >> sh) + stage) * parts + part) << (sh + 7)) + (j << 7) + r;
}

__device__ __forceinline__ void tf_store_chunk(float* a, long long tile, int kc, int r, int K4, int KC, int parts, const float v[4]) {
    float hi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) hi[j] = round_tf32(v[j]);
    reinterpret_cast<float4*>(a)[tf_chunk_index(tile, kc, 0, r, K4, KC, parts)] = make_float4(hi[0], hi[1], hi[2], hi[3]);
    if (parts == 2) {
        float lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) lo[j] = round_tf32(__fsub_rn(v[j], hi[j]));
        reinterpret_cast<float4*>(a)[tf_chunk_index(tile, kc, 1, r, K4, KC, parts)] = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// A[(n, oh, ow)][k], k = (c, kh, kw) in that order, in the blocked layout; taps outside the image and the K padding
// are zero.  One CTA per row tile: a thread owns one of the tile's 128 rows (its pixel is decoded once) and walks the
// K chunks; where each k reads is a table built on the host (no division in the loop).  A warp's 32 lanes read 32
// consecutive pixels of one tap and write 512 contiguous bytes.
__global__ void __launch_bounds__(256) im2col_f32_blocked_kernel(const TfIm2colArgs p) {
    const ConvGeom& g = p.g;
    const int tid = threadIdx.x, r = tid & 127;
    const long long n_tiles = (p.rows + 127) / 128;
    const long long plane = (long long)g.H * g.W;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row = tile * 128 + r;
        const bool row_ok = row < p.rows;
        int ih0 = 0, iw0 = 0;
        long long base = 0;
        if (row_ok) {
            const int ow = (int)(row % g.OW); const long long t = row / g.OW;
            const int oh = (int)(t % g.OH); const long long n = t / g.OH;
            ih0 = oh * g.sh - g.pt; iw0 = ow * g.sw - g.pl;
            base = n * g.C * plane + (long long)ih0 * g.W + iw0;
        }
        for (int kc = tid >> 7; kc < p.K4; kc += 2) {
            float vals[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (row_ok) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int2 e = __ldg(p.ktab + kc * 4 + j);            // the same entry for the whole warp
                    const int dy = e.y & 0xffff, dx = e.y >> 16;
                    if (e.y >= 0 && (unsigned)(ih0 + dy) < (unsigned)g.H && (unsigned)(iw0 + dx) < (unsigned)g.W) vals[j] = __ldg(p.x + base + e.x);
                }
            }
            tf_store_chunk(p.a, tile, kc, r, p.K4, p.KC, p.parts, vals);
        }
    }
}

// A row-major (or transposed) matrix [M][K] with element strides (sm, sk) -> blocked, rounded to TF32.
__global__ void __launch_bounds__(256) block_matrix_f32_kernel(const float* __restrict__ x, float* __restrict__ a, long long M, int K, int K4,
                                                               long long sm, long long sk, int KC, int parts) {
    const long long rows_pad = (M + 127) / 128 * 128;
    const long long total = rows_pad * K4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i & 127);
        const long long tk = i >> 7;
        const int kc = (int)(tk % K4);
        const long long tile = tk / K4;
        const long long row = tile * 128 + r;
        float vals[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (row < M) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = kc * 4 + j;
                if (k < K) vals[j] = __ldg(x + row * sm + (long long)k * sk);
            }
        }
        tf_store_chunk(a, tile, kc, r, K4, KC, parts, vals);
    }
}

// Host-side preparation of the right operand (weights) of one contraction.
struct TfGemmPrep {
    int NT = 0, N_pad = 0, n_out = 0, K = 0, K4 = 0;
    int KC = 8, parts = 1;         // chunks of K per pipeline stage (8 = 32 floats; 4 in the split form); 2 parts = hi and lo
    std::vector<float> w_blk;      // [N_pad/NT][K4/KC][parts][KC][NT][4], rounded to TF32
    std::vector<float> bias;       // [N_pad]
    std::vector<int32_t> ktab;     // convolutions: [K4 * 4][2], where each k of the im2col row reads (see TfIm2colArgs)
};

inline float host_round_tf32(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7f800000u) != 0x7f800000u) { u += 0x00001000u; }     // nearest, ties away from zero (finite values)
    u &= 0xffffe000u;
    float r;
    std::memcpy(&r, &u, 4);
    return r;
}

// w(n, k) = w[n * sn + k * sk]: a convolution's [M][C][KH][KW] weight is (sn = K, sk = 1); a MatMul's B [K][N] is (1, N).
// `split`: the 3 x TF32 form (hi and lo parts of both operands).
inline void tf_gemm_prepare(const float* w, int n_out, int K, long long sn, long long sk, const float* bias, TfGemmPrep& p, long long rows = 0, bool split = false) {
    p.parts = split ? 2 : 1;
    p.KC = split ? 4 : 8;
    p.NT = n_out <= 64 ? 64 : (n_out <= 128 ? 128 : 256);
    if (p.NT == 256 && rows > 0) {
        const long long mt = (rows + 127) / 128;
        const long long t256 = mt * ((n_out + 255) / 256), t128 = mt * ((n_out + 127) / 128);
        if ((t128 + 147) / 148 * 128 < (t256 + 147) / 148 * 256) p.NT = 128;
    }
    p.n_out = n_out;
    p.N_pad = (n_out + p.NT - 1) / p.NT * p.NT;
    p.K = K;
    p.K4 = (K + 4 * p.KC - 1) / (4 * p.KC) * p.KC;
    p.w_blk.assign((size_t)p.N_pad * p.K4 * 4 * p.parts, 0.0f);
    p.bias.assign(p.N_pad, 0.0f);
    for (int n = 0; n < n_out; ++n) {
        float* tile = p.w_blk.data() + (size_t)(n / p.NT) * p.K4 * p.parts * p.NT * 4;
        for (int k = 0; k < K; ++k) {
            const int kc = k >> 2, stage = kc / p.KC, j = kc % p.KC;
            const float v = w[n * sn + k * sk];
            const float hi = host_round_tf32(v);
            const size_t at = (((size_t)stage * p.parts) * p.KC + j) * p.NT * 4 + (size_t)(n % p.NT) * 4 + (k & 3);
            tile[at] = hi;
            if (split) tile[at + (size_t)p.KC * p.NT * 4] = host_round_tf32(v - hi);
        }
        if (bias) p.bias[n] = bias[n];
    }
}

// The gather table of a convolution's im2col rows: k = (c, kh, kw) in the weight tensor's order.
inline void tf_conv_table(const ConvGeom& g, TfGemmPrep& p) {
    p.ktab.assign((size_t)p.K4 * 4 * 2, -1);
    const int khw = g.KH * g.KW;
    for (int k = 0; k < p.K; ++k) {
        const int c = k / khw, tap = k % khw, kh = tap / g.KW, kw = tap % g.KW;
        p.ktab[2 * k] = c * g.H * g.W + kh * g.dh * g.W + kw * g.dw;
        p.ktab[2 * k + 1] = (kh * g.dh) | ((kw * g.dw) << 16);
    }
}

inline size_t tf_gemm_a_bytes(size_t rows, const TfGemmPrep& p) { return (rows + 127) / 128 * 128 * (size_t)p.K4 * 16 * p.parts; }

template <int NT, bool SPLIT>
inline int32_t launch_tf_gemm(zant_ctx* ctx, const TfGemmArgs& k, int tiles) {
    constexpr int STAGES = NT == 256 ? 4 : 6;
    constexpr int KC = SPLIT ? 4 : 8;          // the same bytes per stage in both forms
    using Cfg = TfGemmCfg<NT, KC, STAGES, SPLIT>;
    ZB_SMEM_ATTR(ctx, (tc_gemm_tf32_kernel<NT, KC, STAGES, SPLIT>), Cfg::SMEM_BYTES);
    tc_gemm_tf32_kernel<NT, KC, STAGES, SPLIT><<<std::min(tiles, ctx->sm_count), Cfg::THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(k);
    return check_launch(ctx, SPLIT ? "tc_gemm_tf32_kernel<split>" : "tc_gemm_tf32_kernel");
}

// GEMM on a blocked left operand.  `ohw` > 0 stores NCHW (rows = (image, position)), 0 stores row-major [M][n_out].
inline int32_t run_tf_gemm(zant_ctx* ctx, const TfGemmPrep& p, const float* a_blk, const float* w_blk_dev, const float* bias_dev, long long M,
                           int ohw, int act, float slope, float* y) {
    if (M <= 0) return ZANT_OK;
    if (M > 0x7fffffffLL - 128 || p.N_pad > TfGemmCfg<64, 8, 4>::MAX_N) return fail(ZANT_E_TOO_LARGE, "TF32 GEMM dimensions");
    TfGemmArgs k{};
    k.a = a_blk; k.w = w_blk_dev; k.bias = bias_dev; k.y = y; k.M = (int)M; k.N = p.N_pad; k.K4 = p.K4; k.n_valid = p.n_out; k.ohw = ohw;
    k.act = act; k.slope = slope; k.status = ctx->status_word;
    const long long tiles_ll = (M + 127) / 128 * (p.N_pad / p.NT);
    if (tiles_ll > 0x7fffffffLL) return fail(ZANT_E_TOO_LARGE, "TF32 GEMM tiles");
    const int tiles = (int)tiles_ll;
    if (p.parts == 2) {
        if (p.NT == 64) return launch_tf_gemm<64, true>(ctx, k, tiles);
        if (p.NT == 128) return launch_tf_gemm<128, true>(ctx, k, tiles);
        return launch_tf_gemm<256, true>(ctx, k, tiles);
    }
    if (p.NT == 64) return launch_tf_gemm<64, false>(ctx, k, tiles);
    if (p.NT == 128) return launch_tf_gemm<128, false>(ctx, k, tiles);
    return launch_tf_gemm<256, false>(ctx, k, tiles);
}

// Convolution (group 1, any stride / dilation / padding): im2col gather + GEMM.  `a_blk` is scratch of tf_gemm_a_bytes(N*OH*OW).
inline int32_t run_conv_tf32(zant_ctx* ctx, const ConvGeom& g, const float* x, const TfGemmPrep& p, const float* w_blk_dev, const float* bias_dev,
                             const int32_t* ktab_dev, float* a_blk, int act, float slope, float* y) {
    TfIm2colArgs ia{};
    ia.x = x; ia.a = a_blk; ia.g = g; ia.rows = (long long)g.N * g.OH * g.OW; ia.K = p.K; ia.K4 = p.K4; ia.KC = p.KC; ia.parts = p.parts;
    if (ia.rows <= 0) return ZANT_OK;
    ia.ktab = reinterpret_cast<const int2*>(ktab_dev);
    if ((long long)g.C * g.H * g.W > 0x7fffffffLL || g.KH * g.dh > 0x7fff || g.KW * g.dw > 0x7fff) return fail(ZANT_E_TOO_LARGE, "convolution geometry exceeds the gather table's range");
    const long long n_tiles = (ia.rows + 127) / 128;
    im2col_f32_blocked_kernel<<<(unsigned)std::min<long long>(n_tiles, (long long)ctx->sm_count * 16), 256, 0, ctx->stream>>>(ia);
    ZB_TRY(check_launch(ctx, "im2col_f32_blocked_kernel"));
    return run_tf_gemm(ctx, p, a_blk, w_blk_dev, bias_dev, ia.rows, g.OH * g.OW, act, slope, y);
}

// Matrix product with a strided left operand: blocks A, then the GEMM; row-major result.
inline int32_t run_matmul_tf32(zant_ctx* ctx, const float* a, long long M, int K, long long sm, long long sk, const TfGemmPrep& p,
                               const float* w_blk_dev, const float* bias_dev, float* a_blk, int act, float slope, float* y) {
    if (M <= 0) return ZANT_OK;
    const long long chunks = (M + 127) / 128 * 128 * (long long)p.K4;
    block_matrix_f32_kernel<<<grid_for((size_t)chunks, 256, ctx->sm_count, 16), 256, 0, ctx->stream>>>(a, a_blk, M, K, p.K4, sm, sk, p.KC, p.parts);
    ZB_TRY(check_launch(ctx, "block_matrix_f32_kernel"));
    return run_tf_gemm(ctx, p, a_blk, w_blk_dev, bias_dev, M, 0, act, slope, y);
}

}  // namespace zb
