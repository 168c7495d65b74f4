// int8 GEMM on tcgen05 for fully-connected layers:  Y[M,N] = requant(A[M,K] * W[K,N] + bias).
//
// Operand layout "GEMM-blocked": rows are grouped in tiles (128 rows of A, NT rows of W^T) and
// inside a tile K is split into 16-byte chunks, chunk-major:  [tile][K/16][rows][16] int8.  A run
// of chunks of one tile is therefore contiguous in global memory — one bulk async copy per
// operand and pipeline stage, no tensor map — and lands in shared memory directly in the
// K-major, no-swizzle form tcgen05 reads (8 rows = 8 consecutive 16-byte chunks; the second
// chunk of a 32-byte MMA K step lies rows*16 bytes further).
//
// Persistent CTAs (one per SM, all 512 TMEM columns: two 128 x 256 int32 accumulators), warp roles:
//   warp 0    producer: bulk copies of A and W stages (KC chunks of K each), STAGES-deep ring
//   warp 1    TMEM owner + MMA issuer: KC/2 MMAs (128 x NT x 32) per stage
//   warps 2-9 epilogue (each lane quarter is served by two warps that split the tile's columns):
//             TMEM -> registers, + bias, requantise (per-column constants from shared memory),
//             ReLU, store
// Tile order: t -> (m = t / n_tiles, n = t % n_tiles), so CTAs that run at the same time share
// their A tile through L2.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "fused_cnn.cuh"
#include "kernels_q8.cuh"
#include "ptx_sm100.cuh"

namespace zb {

struct TcGemmArgs {
    const int8_t* a;       // [ceil(M/128)][K16][128][16]
    const int8_t* w;       // [N/NT][K16][NT][16]
    const float* mult;     // [N]
    const int32_t* bias;   // [N]
    int8_t* y;             // [M][N] row-major
    int M, N, K16;         // N = padded column count (multiple of NT), K16 = K/16, a multiple of KC
    float y_scale; int y_zp; int act;
    const uint8_t* lut;       // MODE 2 only: optional table applied to the output codes (see Requant)
    int* status;
    // MODE & 2 (convolution output): valid columns (output channels), positions per image (OH*OW)
    // and output type; rows are (image, position) and the result is stored NCHW.
    int n_valid; int ohw; int out_u8;
    // MODE & 2: int8 output with zero point 0 and finite multipliers (host-checked): requantisation by rni and a saturating
    // pack, the activation as a clamp of the packed codes to [0 | -128, six | 127]
    int lean; int six;
};

template <int NT, int KC, int STAGES, int MODE = 0>
struct TcGemmCfg {
    static constexpr int A_STAGE = KC * 128 * 16;
    static constexpr int W_STAGE = KC * NT * 16;
    static constexpr int STAGE = A_STAGE + W_STAGE;
    static constexpr int MAX_N = 2048;                       // per-column constants kept in shared memory
    static constexpr int OFF_STAGES = 0;
    static constexpr int OFF_CONST = OFF_STAGES + STAGES * STAGE;   // float mult[MAX_N]; int bias[MAX_N]
    static constexpr int OFF_BAR = OFF_CONST + 2 * MAX_N * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 512;
    static constexpr int TMEM_COLS = 2 * NT;
    // warps per TMEM lane quarter (they split the tile's columns): two for the row-major epilogue, which is bound by the
    // operand feed anyway; four for the NCHW-storing one (with two per scheduler it was latency-bound: 35 % issue-active)
    static constexpr int PARTS = ((MODE & 2) && NT >= 128) ? 4 : 2;
    static constexpr int COLS_PER_WARP = NT / PARTS;
    static constexpr int EPI_WARPS = 4 * PARTS;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;      // producer, MMA issuer, epilogue warps
    static_assert(KC % 2 == 0, "a stage must hold whole 32-byte MMA K steps");
    static_assert(NT % 64 == 0 && NT <= 256, "tile width");
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");
    static_assert(2 * STAGES + 4 <= 48, "barrier slots");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// Requires: int8 output with zero point 0, positive finite multipliers, N <= MAX_N (host-checked).
// MODE bit 0: A holds uint8 (else int8).  MODE bit 1: general requantisation (any zero point,
// int8 or uint8, ReLU / ReLU6) and NCHW store; otherwise the lean int8 / zero-point-0 form with a
// row-major [M][N] store.
template <int NT, int KC, int STAGES, int MODE = 0>
__global__ void __launch_bounds__(TcGemmCfg<NT, KC, STAGES, MODE>::THREADS, 1) tc_gemm_i8_kernel(const __grid_constant__ TcGemmArgs a) {
    using Cfg = TcGemmCfg<NT, KC, STAGES, MODE>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sStages = smem + Cfg::OFF_STAGES;
    float* sMult = reinterpret_cast<float*>(smem + Cfg::OFF_CONST);
    int* sBias = reinterpret_cast<int*>(smem + Cfg::OFF_CONST + Cfg::MAX_N * 4);
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
    const int k_stages = a.K16 / KC;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(full(s), 1); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), Cfg::EPI_WARPS); }
        *abort_flag = 0;
        *epi_ok = 1;
        ptx::mbar_fence_init();
    }
    for (int i = tid; i < a.N; i += Cfg::THREADS) { sMult[i] = __ldg(a.mult + i); sBias[i] = __ldg(a.bias + i); }
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
                const int8_t* ga = a.a + (size_t)m * a.K16 * 2048;
                const int8_t* gw = a.w + (size_t)n * a.K16 * (NT * 16);
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) goto producer_done;
                    ptx::mbar_arrive_expect_tx(full(s), Cfg::STAGE);
                    const uint32_t dst = ptx::smem_u32(sStages + s * Cfg::STAGE);
                    ptx::bulk_g2s(dst, ga + (size_t)ks * Cfg::A_STAGE, Cfg::A_STAGE, full(s));
                    ptx::bulk_g2s(dst + Cfg::A_STAGE, gw + (size_t)ks * Cfg::W_STAGE, Cfg::W_STAGE, full(s));
                }
            }
        producer_done:;
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(128, NT, (MODE & 1) == 0, true);
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
                    const uint32_t sa = ptx::smem_u32(sStages + s * Cfg::STAGE);
                    const uint32_t sw = sa + Cfg::A_STAGE;
#pragma unroll
                    for (int kk = 0; kk < KC / 2; ++kk) {
                        const uint64_t da = ptx::smem_desc_kmajor(sa + (uint32_t)(kk * 2 * 2048), 2048, 128);
                        const uint64_t db = ptx::smem_desc_kmajor(sw + (uint32_t)(kk * 2 * NT * 16), NT * 16, 128);
                        ptx::mma_i8(d_tmem, da, db, idesc, (ks | kk) != 0);
                    }
                    ptx::mma_commit(empty(s));
                }
                ptx::mma_commit(tfull(b));
            }
        mma_done:;
        }
    } else {
        // ------------------------------------------------------------------ epilogue: 8 warps; warp (2+q) and (6+q)
        // read lane quarter q; the first four warps take the tile's left half of the columns.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;            // which part of the tile's columns (0 .. PARTS - 1)
        const int row = quarter * 32 + lane;
        const int e = (warp - 2) * 32 + lane;     // 0 .. 32 * EPI_WARPS - 1
        const bool relu = a.act == ZANT_QACT_RELU;
        int tile_it = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
            const int m = t / n_tiles, n = t - m * n_tiles;
            const int b = tile_it & 1;
            const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
            if (e == 0) *epi_ok = ptx::mbar_wait(tfull(b), bph, abort_flag) ? 1 : 0;
            ptx::named_barrier_sync(1, 32 * Cfg::EPI_WARPS);
            if (!*epi_ok) break;
            ptx::tc_fence_after();
            const int tcol0 = half * Cfg::COLS_PER_WARP;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * NT + tcol0);
            const int grow = m * 128 + row;
            if constexpr ((MODE & 2) == 0) {
                int8_t* yrow = a.y + (size_t)grow * a.N + (size_t)n * NT + tcol0;
#pragma unroll 1
                for (int h = 0; h < Cfg::COLS_PER_WARP / 32; ++h) {
                    uint32_t v[32];
                    ptx::tmem_ld32(taddr + (uint32_t)(h * 32), v);
                    ptx::tmem_wait_ld();
                    const int col0 = n * NT + tcol0 + h * 32;
                    uint32_t packed[8];
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        const float4 m4 = *reinterpret_cast<const float4*>(sMult + col0 + j4 * 4);
                        const int4 b4 = *reinterpret_cast<const int4*>(sBias + col0 + j4 * 4);
                        const int q0 = rq_round((int)v[j4 * 4 + 0] + b4.x, m4.x);
                        const int q1 = rq_round((int)v[j4 * 4 + 1] + b4.y, m4.y);
                        const int q2 = rq_round((int)v[j4 * 4 + 2] + b4.z, m4.z);
                        const int q3 = rq_round((int)v[j4 * 4 + 3] + b4.w, m4.w);
                        const uint32_t pk = pack_sat_s8x4(q0, q1, q2, q3);
                        packed[j4] = relu ? relu_s8x4(pk) : pk;
                    }
                    if (grow < a.M) {
                        reinterpret_cast<uint4*>(yrow + h * 32)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        reinterpret_cast<uint4*>(yrow + h * 32)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    }
                }
            } else {
                // rows are (image, position): consecutive lanes hold consecutive positions, so for a
                // fixed channel a warp writes 32 consecutive bytes of the NCHW output
                const Requant rq{a.y_scale, a.y_zp, a.act, a.lut};
                const int img = grow / a.ohw, pos = grow - img * a.ohw;
                uint8_t* ybase = reinterpret_cast<uint8_t*>(a.y) + (size_t)img * a.n_valid * a.ohw + pos;
                const uint32_t hi4 = a.act == ZANT_QACT_RELU6 ? 0x01010101u * (uint32_t)(a.six & 255) : 0x7f7f7f7fu;
#pragma unroll 1
                for (int h = 0; h < Cfg::COLS_PER_WARP / 32; ++h) {
                    const int col0 = n * NT + tcol0 + h * 32;
                    if (col0 >= a.n_valid) break;                 // the tile's remaining columns are padding
                    uint32_t v[32];
                    ptx::tmem_ld32(taddr + (uint32_t)(h * 32), v);
                    ptx::tmem_wait_ld();
                    if (a.lean) {
                        // four columns at a time: constants as vectors, one saturating pack, the activation on the packed word;
                        // the common case (a row of the matrix, 32 real columns) stores without per-byte tests, the plane
                        // stride kept in registers
                        uint8_t* yc = ybase + (size_t)col0 * a.ohw;
                        const size_t st1 = (size_t)a.ohw, st2 = 2 * st1, st3 = 3 * st1, st4 = 4 * st1;
                        const bool row_ok = grow < a.M, all_cols = col0 + 32 <= a.n_valid;
                        const bool relu_act = a.act != ZANT_QACT_NONE;
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const float4 m4 = *reinterpret_cast<const float4*>(sMult + col0 + j4 * 4);
                            const int4 b4 = *reinterpret_cast<const int4*>(sBias + col0 + j4 * 4);
                            const int q0 = rq_round((int)v[j4 * 4 + 0] + b4.x, m4.x), q1 = rq_round((int)v[j4 * 4 + 1] + b4.y, m4.y);
                            const int q2 = rq_round((int)v[j4 * 4 + 2] + b4.z, m4.z), q3 = rq_round((int)v[j4 * 4 + 3] + b4.w, m4.w);
                            uint32_t w4 = relu_act ? __vminu4(pack_sat_u8x4(q0, q1, q2, q3), hi4) : pack_sat_s8x4(q0, q1, q2, q3);
                            if (a.lut) w4 = lut4(a.lut, w4);
                            if (row_ok && all_cols) {
                                yc[0] = (uint8_t)w4; yc[st1] = (uint8_t)(w4 >> 8); yc[st2] = (uint8_t)(w4 >> 16); yc[st3] = (uint8_t)(w4 >> 24);
                            } else if (row_ok) {
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    if (col0 + j4 * 4 + i < a.n_valid) yc[(size_t)i * st1] = (uint8_t)(w4 >> (8 * i));
                            }
                            yc += st4;
                        }
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = col0 + j;
                        const int acc = (int)v[j] + sBias[col];
                        const int q = a.out_u8 ? requant_one<true>(acc, sMult[col], rq) : requant_one<false>(acc, sMult[col], rq);
                        if (grow < a.M && col < a.n_valid) ybase[(size_t)col * a.ohw] = (uint8_t)q;
                    }
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

// =============================================================================================
// Last layer: QLinearMatMul(K -> NCLS <= 64 classes) + DequantizeLinear, one row per thread.
//   y[row][n] = float(sat(rne(float(acc + bias[n]) * mult[n]) + zp) - zp_dq) * scale_dq
// The weight matrix (K x NCLS int8) is re-packed into shared memory as [NCLS][K/4] words so that
// all threads of a warp read the same word (broadcast) while each walks its own row of A (staged in
// shared memory by coalesced copies).
// =============================================================================================
struct FcOutArgs {
    const int8_t* a;        // [M][K] row-major int8
    const int8_t* w;        // [K][NCLS] int8 (graph layout)
    const float* mult; const int32_t* bias;   // bias already holds -a_zp * sum_k w[k][n]
    float* y;               // [M][NCLS]
    int M, K, NCLS;
    float y_scale; int y_zp;      // requantisation of the int8 logits
    float dq_scale; int dq_zp;    // DequantizeLinear
};

// One warp per tile of 16 rows: the tile (16 x K bytes, contiguous in global memory) is brought into one of the
// warp's two shared-memory buffers with 16-byte cp.async copies (coalesced; the next tile's copies are in flight
// while the current tile is multiplied), rows padded by 16 bytes so that the fragment loads hit distinct banks.
// Only __syncwarp between the phases: warps run independently and the grid balances at 16-row granularity.
constexpr int FCOUT_THREADS = 128;
template <int K> __host__ __device__ constexpr int fcout_pitch() { return K + 16; }
template <int NC, int K> constexpr int fcout_smem_bytes() { return NC * K + (FCOUT_THREADS / 32) * 32 * fcout_pitch<K>(); }

// The products run on warp-level int8 MMAs (mma.sync m16n8k32, s8 x s8 -> s32): a 32-row tile is two row blocks of 16,
// the classes are NC / 8 column blocks of 8 (weights of classes beyond NCLS are zero), and the B fragments of all K / 32
// steps stay in registers for the whole kernel.  Per tile and warp that is K/32 * 2 * (4 shared-memory loads + NC/8 MMAs)
// instead of 40 dp4a per row and 16 bytes.
template <int NC, int K>   // NC: compile-time bound on the number of classes, a multiple of 8
__global__ void __launch_bounds__(FCOUT_THREADS) fc_out_dequant_kernel(const FcOutArgs p) {
    extern __shared__ __align__(16) uint8_t fc_smem[];
    uint32_t* sw = reinterpret_cast<uint32_t*>(fc_smem);   // [NC][K/4]: word (n, k4) = weights of class n for k = 4*k4 .. 4*k4+3
    constexpr int kw = K / 4, K16 = K / 16, KS = K / 32, NB = NC / 8, PITCH = fcout_pitch<K>();
    static_assert(K % 32 == 0 && K16 <= 32 && 32 % K16 == 0 && NC % 8 == 0, "K: whole MMA steps, a row of 1..32 16-byte chunks; NC: whole column blocks");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint8_t* sa = fc_smem + NC * K + warp * 32 * PITCH;       // this warp's [32][PITCH]
    for (int i = threadIdx.x; i < NC * kw; i += blockDim.x) {
        const int n = i / kw, k4 = i - n * kw;
        uint32_t word = 0;
        if (n < p.NCLS)
            for (int j = 0; j < 4; ++j) word |= (uint32_t)(uint8_t)p.w[(size_t)(k4 * 4 + j) * p.NCLS + n] << (8 * j);
        sw[i] = word;
    }
    __syncthreads();
    // B fragments: column g of block nb, k = 32*ks + 4t .. +3 and 32*ks + 16 + 4t .. +3
    uint32_t bf[NB][KS][2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            bf[nb][ks][0] = sw[(nb * 8 + g) * kw + ks * 8 + t];
            bf[nb][ks][1] = sw[(nb * 8 + g) * kw + ks * 8 + 4 + t];
        }
    // this lane's output columns (2t, 2t+1 of every block) and their constants
    float mult[NB][2]; int bias[NB][2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int col = nb * 8 + 2 * t + c;
            mult[nb][c] = col < p.NCLS ? __ldg(p.mult + col) : 0.0f;
            bias[nb][c] = col < p.NCLS ? __ldg(p.bias + col) : 0;
        }
    const Requant rq{p.y_scale, p.y_zp, ZANT_QACT_NONE};
    const int tiles = (p.M + 15) / 16;                        // tiles of 16 rows, two buffers per warp: the next tile's copy
    const int warps_total = gridDim.x * (FCOUT_THREADS / 32);  // is in flight while the current one is multiplied
    constexpr int ROWS_PER_PASS = 32 / K16;                   // rows covered by one copy instruction of the warp
    const int cr = lane / K16, cc = lane - cr * K16;
    auto copy_tile = [&](int tile, int buf) {
        const int row0 = tile * 16, rows = min(16, p.M - row0);
        const int8_t* src = p.a + (size_t)row0 * K;
        uint8_t* dstb = sa + buf * 16 * PITCH;
#pragma unroll 8
        for (int r = cr; r < rows; r += ROWS_PER_PASS) {
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(dstb + r * PITCH + cc * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + (size_t)r * K + cc * 16) : "memory");
        }
    };
    int tile = blockIdx.x * (FCOUT_THREADS / 32) + warp, buf = 0;
    if (tile < tiles) copy_tile(tile, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (; tile < tiles; tile += warps_total, buf ^= 1) {
        if (tile + warps_total < tiles) copy_tile(tile + warps_total, buf ^ 1);
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 1;" ::: "memory");      // everything but the newest group has landed
        __syncwarp();
        const int row0 = tile * 16, rows = min(16, p.M - row0);
        const uint8_t* sb = sa + buf * 16 * PITCH;
        int acc[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0;
        const uint32_t* r_lo = reinterpret_cast<const uint32_t*>(sb + g * PITCH) + t;          // rows past the tile's end hold stale bytes
        const uint32_t* r_hi = reinterpret_cast<const uint32_t*>(sb + (g + 8) * PITCH) + t;    // and are not stored
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint32_t a0 = r_lo[ks * 8], a1 = r_hi[ks * 8], a2 = r_lo[ks * 8 + 4], a3 = r_hi[ks * 8 + 4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
                asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+r"(acc[nb][0]), "+r"(acc[nb][1]), "+r"(acc[nb][2]), "+r"(acc[nb][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(bf[nb][ks][0]), "r"(bf[nb][ks][1]));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {                         // accumulators 0,1: row g; 2,3: row g + 8
            const int r = g + 8 * h;
            if (r < rows) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int col = nb * 8 + 2 * t + c;
                        if (col < p.NCLS) {
                            const int q = requant_one<false>(acc[nb][2 * h + c] + bias[nb][c], mult[nb][c], rq);
                            p.y[(size_t)(row0 + r) * p.NCLS + col] = __fmul_rn(__int2float_rn(q - p.dq_zp), p.dq_scale);
                        }
                    }
            }
        }
        __syncwarp();      // the tile's reads are done before the copy after next overwrites it
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

}  // namespace zb
