// Pointwise (1x1, stride 1, no padding, group 1) QLinearConv on tcgen05 with the FILTERS on the accumulator's lanes.
//
// Per image a 1x1 convolution is the product  Y[M filters][HW pixels] = W[M][C] . X[C][HW].  With NCHW tensors both X
// and Y keep the pixel index contiguous, so the natural tcgen05 form is
//     D (TMEM: lane = filter, column = pixel)  =  A (weights [128 filters][K], K-major)  x  B (activations, N-major),
// where the B operand of a stage is a box [K chunk][128 pixels] of the input exactly as it lies in memory: a tiled TMA
// load with the 128-byte swizzle drops it into shared memory in the "MN-major" operand form, nothing is transposed.
// In the epilogue a thread owns one filter and reads 32 consecutive pixels of it from TMEM: the multiplier and bias are
// two registers, four results pack into one word, and the 32 bytes leave as one 32-byte store into the filter's NCHW
// plane.  (The implicit-GEMM kernel for k x k filters puts pixels on the lanes and has to transpose bytes through
// shared memory on the way out; for 1x1 filters this form has neither that nor a patch to build.)
//
// A CTA keeps the weights of ONE tile of 128 filters resident in shared memory (K <= 960) and walks over (image,
// pixel tile) pairs; a pixel tile is up to 256 pixels (two accumulator buffers of 256 TMEM columns each, so the
// epilogue of a tile overlaps the MMAs of the next).
// Planes whose size is a multiple of 4 but not of 16 bytes (14 x 14) have no tensor map.  A stage's channel rows are one
// contiguous, 16-byte aligned run of the input, so the loader brings them in with one 1-D bulk copy per stage into a ring of
// raw buffers, and four copier warps re-lay a raw buffer out into the swizzled operand form with shared-memory word loads and
// stores (copying from global memory with plain loads left the kernel waiting on their latency: too few bytes in flight).
// The output tile - for a whole image the block [128 filters][HW] is contiguous in NCHW - is staged in shared memory and
// leaves as one bulk copy.
//
// Few filters (at most 64): a tile of 128 lanes would leave lane quarters idle, and the epilogue - the part that bounds the
// kernel - would run on one or two of the SM's four schedulers.  The lanes then carry G = 128 / m_pad GROUPS of m_pad filters,
// each group working on its own run of pixels: A is block-diagonal, [group g][filter] x [group g'][channel] = W[filter][channel]
// for g == g' and zero elsewhere, K is G times as deep, and K iteration (g', channel chunk) loads the TMA box of group g''s
// pixels.  The zero blocks cost MMA time, of which there is plenty; every lane of the epilogue has work.
//
// 3x3 stems (mode 2; at most three input channels, stride 1 or 2, at most 64 filters): K = 9 * cin <= 27 is one K step, the filters
// run as pixel groups on the lanes, and the B operand of a group - row k = (channel, kh, kw), column = output pixel - is written
// by the copier warps: the loader brings the input rows of a tile's output rows into a raw buffer (one bulk copy per channel),
// a copier lane cuts the 16-byte chunks (16 output pixels) of the three taps of a filter row out of the 16 * stride + 2 input
// bytes it read once (funnel shifts; stride 2: every second byte by byte permutes), replaces what lies outside the image by the
// input zero point and stores the chunks at their swizzled places; each copier warp builds every fourth pixel group on its own
// (pw_stem_builder).  That is an im2col matrix which only ever exists in shared memory, 27 bytes per output pixel for all filters.
//
// Warp roles (704 threads, one persistent CTA per SM):
//   warp 0  loader (TMA boxes or bulk copies)     warp 1  TMEM owner + MMA issuer     warps 2-17  epilogue
//   warps 18-21  copiers (small planes: re-layout of the raw rows; stems: builders of the patch operand)
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "context.cuh"
#include "fused_cnn.cuh"
#include "geometry.hpp"
#include "kernels_q8.cuh"
#include "ptx_sm100.cuh"

namespace zb {

struct PwConvArgs {
    const uint8_t* x; uint8_t* y; const int8_t* w; const float* mult; const int32_t* bias;
    int N, C, M, HW;
    int k_steps;          // K steps of 32 channels (C rounded up)
    int KS;               // K steps per stage (a stage holds KS * 32 channels)
    int n_px;             // pixels per tile: a multiple of 16, at most 256
    int px_tiles;         // tiles per image
    int PB;               // 128-pixel blocks per tile (1 or 2)
    int G;                // pixel groups on the lanes (1, or 128 / m_pad when there are at most 64 filters: see the kernel's header)
    int m_pad;            // lanes per group: 16, 32 or 64 filters (128 when G == 1)
    int a_steps;          // K steps of the resident A operand: k_steps, or G * (K iterations per group) * KS for the block-diagonal form
    int cpm;              // CTAs per filter tile
    int mode;             // 0: tensor map; 1: bulk copies + re-layout in, staged tile out (HW % 4 == 0, at most 256 pixels: one tile per image);
                          // 2: 3x3 stem, the B operand is built from input rows (see PwConvArgs::cin)
    int bulk_out;         // mode 1: the staged tile leaves as one bulk copy (its address and size are multiples of 16)
    int wide_store;       // mode 0: every 32-pixel chunk starts at a 32-byte boundary (HW and n_px are multiples of 32)
    int stages, stage_bytes, off_stages, off_out, off_tail;
    int outs, out_stride;           // mode 1: staging buffers for the output tile (two when they fit: a tile is staged while the previous one is sent)
    int raws, raw_bytes, off_raw;   // modes 1, 2: ring of raw buffers that bulk copies fill with input rows as they lie in memory
    // mode 2 (3x3 stems: at most three input channels, stride 1 or 2): geometry of the convolution whose patches the builder
    // warps write as the B operand (K = 9 * cin, zero-padded to 32); HW above is the OUTPUT plane OH * OW
    int cin, ih, iw, oh, ow, cs, pt, pl, band;   // input channels, input H and W, output H and W, stride, pads, input rows per raw buffer and channel
    uint32_t pad_word;
    uint32_t ow_magic;    // mode 2: floor(2^32 / ow) + 1; umulhi(p, ow_magic) == p / ow for every pixel index of the plane
    float y_scale; int y_zp; int act; int out_u8; int six;
    const int32_t* cap;   // lean epilogue, act_mode 1: per-filter accumulator bound of the activation (requant_relu_caps)
    int act_mode;         // lean epilogue: 0 no activation, 1 clamp of the accumulator to [0, cap], 2 clamp of the packed codes
    const uint8_t* lut;
    int* status;
};

constexpr int kPwThreads = 704;
constexpr int kPwMaxStages = 8;
constexpr int kPwTail = 1024;                 // barriers, TMEM slot, flags, activation table
constexpr uint32_t kIdescBMnMajor = 1u << 16; // bit 16 of the instruction descriptor: B is MN-major (its N index is the contiguous one)

__device__ __forceinline__ void st_global_32B(uint8_t* p, const uint32_t (&v)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

using ptx::bulk_s2g;
using ptx::bulk_wait_all;
__device__ __forceinline__ void bulk_wait_read() { ptx::bulk_wait_read<0>(); }

// Barrier slots of the kernel below, in 8-byte units from the start of its tail.
__device__ __forceinline__ uint32_t pw_bar_full(uint32_t bar0, int s) { return bar0 + 8u * s; }
__device__ __forceinline__ uint32_t pw_bar_empty(uint32_t bar0, int s) { return bar0 + 8u * (kPwMaxStages + s); }
__device__ __forceinline__ uint32_t pw_bar_raw_full(uint32_t bar0, int r) { return bar0 + 8u * (2 * kPwMaxStages + 5 + r); }
__device__ __forceinline__ uint32_t pw_bar_raw_empty(uint32_t bar0, int r) { return bar0 + 8u * (2 * kPwMaxStages + 9 + r); }

// Shared-memory accesses by 32-bit address (and immediate offset), in program order.
template <int OFF>
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_u128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Stem (mode 2), one of the four builder warps: the B operand of every fourth pixel group of this CTA's tiles (in the order
// the MMA issuer consumes them), from the tiles' raw input rows.  Eight stages, two per warp: warp w builds the groups
// w, w + 4, ... into the stages w, w + 4, w, ..., so four groups are under construction at a time, a warp does not wait for
// the MMA that reads its previous group, and nothing but the mbarriers orders the warps.
// A lane owns a 16-byte chunk of the stage's rows - 16 output pixels of one output row (ow % 16 == 0) - and every second
// (channel, filter row) pair: the 16 * CS + 2 input bytes of the pair's window are read once (one or two 16-byte words and
// the word on either side) and give the chunk in the rows of the three taps kw = 0, 1, 2, each stored as one 16-byte word.
// CS: stride; PL: left padding.  The window of tap kw = 0 starts PL bytes in front of a 16-byte boundary.
template <int CS, int PL>
__device__ __forceinline__ void pw_stem_builder(const PwConvArgs& a, uint32_t smem0, uint32_t bar0, int cw, int lane, int j0, int tiles, int tile_px,
                                                volatile int* abort_flag) {
    constexpr int NX = 4 * CS;                                          // aligned words of the window; X[0] and X[NX + 1] are the neighbours
    const int nc = a.n_px >> 4;                                         // chunks per group
    const int ci = lane & 15, qh = lane >> 4;
    const int plane = a.band * a.iw;                                    // bytes of a channel in a raw buffer
    const int Q = 3 * a.cin;                                            // (channel, filter row) pairs
    const uint32_t pad = a.pad_word;
    const uint32_t ci7 = (uint32_t)ci & 7u, blk = ((uint32_t)ci >> 3) * 4096u;    // chunk in its 128-pixel block, the block
    uint32_t n_built = 0;                                               // groups this warp has built: stage cw + 4 * (n_built % 2)
    int g = 0, tile_it = 0;                                             // groups and tiles of this CTA so far
    for (int t = j0; t < tiles; t += a.cpm, ++tile_it) {
        const int img = t / a.px_tiles, p0 = (t - img * a.px_tiles) * tile_px;
        const int ih_lo = (int)__umulhi((uint32_t)p0, a.ow_magic) * CS - a.pt;
        const int r = tile_it % a.raws;
        const uint32_t rph = (uint32_t)(tile_it / a.raws) & 1u;
        // +16: the word in front of the first row is read
        const uint32_t raw = smem0 + (uint32_t)(a.off_raw + r * a.raw_bytes + 16);
#pragma unroll 1
        for (int pg = 0; pg < a.G; ++pg, ++g) {
            if ((g & 3) != cw) continue;
            const int st = cw + 4 * (int)(n_built & 1u);                // the ring has eight stages: group g lives in stage g % 8
            int ok = 1;
            if (lane == 0)
                ok = (ptx::mbar_wait_sleeping(pw_bar_raw_full(bar0, r), rph, abort_flag) &&
                      ptx::mbar_wait_sleeping(pw_bar_empty(bar0, st), ((n_built >> 1) & 1u) ^ 1u, abort_flag)) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) return;
            ++n_built;
            const uint32_t dst = smem0 + (uint32_t)(a.off_stages + st * a.stage_bytes) + blk;
            const int p = p0 + pg * a.n_px + 16 * ci;                   // first of the chunk's 16 output pixels
            const int oy = (int)__umulhi((uint32_t)p, a.ow_magic), ox = p - oy * a.ow;
            const bool act = ci < nc && p < a.HW;                       // (columns past the plane: never stored by the epilogue)
            const int row0 = oy * CS - a.pt;                            // input row of kh = 0
            const uint32_t base = raw + (uint32_t)((row0 - ih_lo) * a.iw + ox * CS);
            const bool left = PL && ox == 0;                            // the first pixel of tap kw = 0 lies left of the image
            const int room = a.iw - 15 * CS - (ox * CS - PL);           // taps kw >= room: the last pixel lies right of it
#pragma unroll 1
            for (int q = qh; q < Q; q += 2) {
                const int c = q / 3, kh = q - 3 * c;
                // rows above and below the image: the zero point
                const bool ld = act && (unsigned)(row0 + kh) < (unsigned)a.ih;
                const uint32_t ad = ld ? base + (uint32_t)(c * plane + kh * a.iw) : raw + 16u;
                uint32_t X[NX + 2];
                {
                    X[0] = lds_u32<0>(ad - 4u);
                    const uint4 A = lds_u128(ad);
                    X[1] = A.x; X[2] = A.y; X[3] = A.z; X[4] = A.w;
                    if (CS == 2) {
                        const uint4 B = lds_u128(ad + 16u);
                        X[5] = B.x; X[6] = B.y; X[7] = B.z; X[8] = B.w;
                    }
                    X[NX + 1] = lds_u32<4 * NX>(ad);
                }
                if (!ld) {
#pragma unroll
                    for (int i = 0; i < NX + 2; ++i) X[i] = pad;
                }
                // word j (four output pixels) of tap kw starts at byte 4 * CS * j + kw - PL of the window; X[1] holds byte 0
                uint32_t v[3][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (CS == 1) {
                        v[0][j] = PL ? __funnelshift_r(X[j], X[j + 1], 24) : X[j + 1];
                        v[1][j] = PL ? X[j + 1] : __funnelshift_r(X[j + 1], X[j + 2], 8);
                        v[2][j] = PL ? __funnelshift_r(X[j + 1], X[j + 2], 8) : __funnelshift_r(X[j + 1], X[j + 2], 16);
                    } else if (PL) {
                        // bytes 8j - 1, + 1, + 3, + 5;  8j, + 2, + 4, + 6;  8j + 1, + 3, + 5, + 7
                        v[0][j] = __byte_perm(__byte_perm(X[2 * j], X[2 * j + 1], 0x0753), X[2 * j + 2], 0x5210);
                        v[1][j] = __byte_perm(X[2 * j + 1], X[2 * j + 2], 0x6420);
                        v[2][j] = __byte_perm(X[2 * j + 1], X[2 * j + 2], 0x7531);
                    } else {
                        // bytes 8j, + 2, + 4, + 6;  8j + 1, + 3, + 5, + 7;  8j + 2, + 4, + 6, + 8
                        v[0][j] = __byte_perm(X[2 * j + 1], X[2 * j + 2], 0x6420);
                        v[1][j] = __byte_perm(X[2 * j + 1], X[2 * j + 2], 0x7531);
                        v[2][j] = __byte_perm(__byte_perm(X[2 * j + 1], X[2 * j + 2], 0x0642), X[2 * j + 3], 0x4210);
                    }
                }
                if (left) v[0][0] = (v[0][0] & 0xffffff00u) | (pad & 0xffu);
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
                    if (kw >= room) v[kw][3] = (v[kw][3] & 0x00ffffffu) | (pad & 0xff000000u);
                    const uint32_t k = 3u * (uint32_t)q + (uint32_t)kw;
                    if (act) sts_u128(dst + k * 128u + ((ci7 ^ (k & 7u)) << 4), v[kw][0], v[kw][1], v[kw][2], v[kw][3]);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) { ptx::mbar_arrive(pw_bar_full(bar0, st)); ptx::mbar_arrive(pw_bar_raw_empty(bar0, r)); }
        }
    }
}

template <bool XU8, bool LEAN>
__global__ void __launch_bounds__(kPwThreads, 1) tc_pw_nchw_kernel(const __grid_constant__ PwConvArgs a, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sA = smem;                                  // [k16][128 filters][16]
    uint8_t* sStages = smem + a.off_stages;
    uint8_t* sOut0 = smem + a.off_out;
    uint8_t* tail = smem + a.off_tail;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 256);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 260);
    volatile int* epi_ok = reinterpret_cast<volatile int*>(tail + 264);
    volatile int* cp_ok = reinterpret_cast<volatile int*>(tail + 268);
    uint8_t* sLut = tail + 512;
    const uint32_t bar0 = ptx::smem_u32(bars);
    const int S = a.stages;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kPwMaxStages + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * kPwMaxStages + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * kPwMaxStages + 2 + b); };
    const uint32_t wfull = bar0 + 8u * (2 * kPwMaxStages + 4);
    auto raw_full = [&](int r) { return bar0 + 8u * (2 * kPwMaxStages + 5 + r); };
    auto raw_empty = [&](int r) { return bar0 + 8u * (2 * kPwMaxStages + 9 + r); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mt = (int)blockIdx.x / a.cpm, j0 = (int)blockIdx.x - mt * a.cpm;
    const int tiles = a.N * a.px_tiles;
    const int KC = a.KS * 32;
    const int k_iters = (a.k_steps + a.KS - 1) / a.KS;          // K iterations (stages) per pixel group
    const int k_total = a.G * k_iters;                          // K iterations of a tile
    const int tile_px = a.G * a.n_px;                           // pixels of a tile
    const uint32_t blk_bytes = (uint32_t)KC * 128u;
    const int live_q = a.G > 1 ? 4 : min(4, (a.M - mt * 128 + 31) >> 5);   // lane quarters of this CTA's tile that carry filters

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { ptx::mbar_init(full(s), 1); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), 4 * live_q); }
        ptx::mbar_init(wfull, 1);
        // (stem: every pixel group's builder warp releases the tile's raw buffer)
        for (int r = 0; r < a.raws; ++r) { ptx::mbar_init(raw_full(r), 1); ptx::mbar_init(raw_empty(r), a.mode == 2 ? a.G : 1); }
        *abort_flag = 0; *epi_ok = 1; *cp_ok = 1;
        ptx::mbar_fence_init();
    }
    if (a.lut && tid < 256) sLut[tid] = __ldg(a.lut + tid);
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ loader: the filter tile's weights once, then (mode 0) one box per stage and block
        if (lane == 0) {
            const uint32_t w_bytes = (uint32_t)a.a_steps * 4096u;
            ptx::mbar_arrive_expect_tx(wfull, w_bytes);
            ptx::bulk_g2s(ptx::smem_u32(sA), a.w + (size_t)mt * w_bytes, w_bytes, wfull);
            if (a.mode == 0) {
                int s = 0; uint32_t ph = 0;
                bool alive = true;
                for (int t = j0; t < tiles && alive; t += a.cpm) {
                    const int img = t / a.px_tiles, p0 = (t - img * a.px_tiles) * tile_px;
                    int pg = 0, ki = 0;                                   // pixel group and channel chunk of the K iteration
                    for (int it = 0; it < k_total; ++it) {
                        if (!ptx::mbar_wait_sleeping(empty(s), ph ^ 1u, abort_flag)) { alive = false; break; }
                        const uint32_t dst = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes);
                        ptx::mbar_arrive_expect_tx(full(s), (uint32_t)a.PB * blk_bytes);
                        for (int blk = 0; blk < a.PB; ++blk)
                            ptx::tma_load_3d(dst + (uint32_t)blk * blk_bytes, &x_map, (p0 + pg * a.n_px + blk * 128) >> 2, ki * KC, img, full(s));
                        if (++s == S) { s = 0; ph ^= 1u; }
                        if (++ki == k_iters) { ki = 0; ++pg; }
                    }
                }
            } else if (a.mode == 2) {
                // stem: the input rows that the tile's output rows read, one bulk copy per channel, into the raw ring
                int r = 0; uint32_t ph = 0;
                bool alive = true;
                for (int t = j0; t < tiles && alive; t += a.cpm) {
                    const int img = t / a.px_tiles, p0 = (t - img * a.px_tiles) * tile_px;
                    const int oh_a = p0 / a.ow, oh_b = min(a.oh - 1, (min(a.HW, p0 + tile_px) - 1) / a.ow);
                    const int ih_lo = oh_a * a.cs - a.pt;                                   // first row of the band (may be -1)
                    const int r0 = max(ih_lo, 0), r1 = min(a.ih, oh_b * a.cs - a.pt + 3);   // rows [r0, r1) exist
                    if (!ptx::mbar_wait_sleeping(raw_empty(r), ph ^ 1u, abort_flag)) { alive = false; break; }
                    const uint32_t bytes = (uint32_t)((r1 - r0) * a.iw);                    // a multiple of 16: iw is
                    ptx::mbar_arrive_expect_tx(raw_full(r), bytes * (uint32_t)a.cin);
                    for (int c = 0; c < a.cin; ++c)
                        ptx::bulk_g2s(ptx::smem_u32(smem + a.off_raw + (size_t)r * a.raw_bytes + 16) + (uint32_t)((c * a.band + (r0 - ih_lo)) * a.iw),
                                      a.x + (((size_t)img * a.cin + c) * a.ih + r0) * a.iw, bytes, raw_full(r));
                    if (++r == a.raws) { r = 0; ph ^= 1u; }
                }
            } else {
                // no tensor map: the stage's channel rows [c_lo, c_lo + KC) of the image, one contiguous run, into the raw ring
                int r = 0; uint32_t ph = 0;
                bool alive = true;
                for (int t = j0; t < tiles && alive; t += a.cpm) {
                    const uint8_t* ximg = a.x + (size_t)t * a.C * a.HW;              // one tile per image
                    for (int ki = 0; ki < k_iters; ++ki) {
                        if (!ptx::mbar_wait_sleeping(raw_empty(r), ph ^ 1u, abort_flag)) { alive = false; break; }
                        const int c_lo = ki * KC;
                        const uint32_t bytes = (uint32_t)(min(KC, a.C - c_lo) * a.HW);     // a multiple of 16: C and HW are multiples of 4
                        ptx::mbar_arrive_expect_tx(raw_full(r), bytes);
                        ptx::bulk_g2s(ptx::smem_u32(smem + a.off_raw + (size_t)r * a.raw_bytes), ximg + (size_t)c_lo * a.HW, bytes, raw_full(r));
                        if (++r == a.raws) { r = 0; ph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            const uint32_t n_blk0 = (uint32_t)min(a.n_px, 128), n_blk1 = (uint32_t)(a.n_px - 128);
            const uint32_t idesc0 = ptx::idesc_i8(128, (int)n_blk0, true, !XU8) | kIdescBMnMajor;
            const uint32_t idesc1 = a.PB > 1 ? (ptx::idesc_i8(128, (int)n_blk1, true, !XU8) | kIdescBMnMajor) : 0u;
            const uint64_t da0 = ptx::smem_desc_kmajor(ptx::smem_u32(sA), 128 * 16, 128);
            int s = 0; uint32_t ph = 0;
            int tile_it = 0;
            if (!ptx::mbar_wait_sleeping(wfull, 0, abort_flag)) goto mma_done;
            for (int t = j0; t < tiles; t += a.cpm, ++tile_it) {
                const int b = tile_it & 1;
                const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
                if (!ptx::mbar_wait_sleeping(tempty(b), bph ^ 1u, abort_flag)) goto mma_done;
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * 256);
                for (int ki = 0; ki < k_total; ++ki) {
                    if (!ptx::mbar_wait_sleeping(full(s), ph, abort_flag)) goto mma_done;
                    ptx::tc_fence_after();
                    const uint32_t stage0 = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes);
                    // B = [channel][128 pixels] rows of 128 bytes: eight channels are 1024 bytes, a K step of 32 channels 4096
                    const uint64_t db0 = ptx::smem_desc_mnmajor_sw128(stage0, blk_bytes, 1024);
                    // (the block-diagonal A holds whole stages of K steps per group, zero where the channels end)
                    const int ks_here = a.G > 1 ? a.KS : min(a.KS, a.k_steps - ki * a.KS);
                    for (int kk = 0; kk < ks_here; ++kk) {
                        const uint64_t da = da0 + (uint64_t)((ki * a.KS + kk) * 256);        // 4096 bytes per K step, in 16-byte units
                        const bool acc = (ki | kk) != 0;
                        ptx::mma_i8(d_tmem, da, db0 + (uint64_t)(kk * 256), idesc0, acc);
                        if (a.PB > 1) ptx::mma_i8(d_tmem + 128u, da, db0 + (uint64_t)((blk_bytes >> 4) + kk * 256), idesc1, acc);
                    }
                    ptx::mma_commit(empty(s));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                ptx::mma_commit(tfull(b));
            }
        mma_done:;
        }
    } else if (warp >= 18) {
        // ------------------------------------------------------------------ copiers (no tensor map): a stage's channels, row by row,
        // into the form a swizzled TMA box has: one 128-byte row per channel and 128-pixel block, 16-byte chunk k of row r at
        // chunk position k ^ (r % 8).  Channels past C are skipped: their weights are zero and any finite byte serves.
        if (a.mode == 2) {
            const int cw = warp - 18;
            const uint32_t smem0 = ptx::smem_u32(smem);
            if (a.cs == 1) {
                if (a.pl) pw_stem_builder<1, 1>(a, smem0, bar0, cw, lane, j0, tiles, tile_px, abort_flag);
                else pw_stem_builder<1, 0>(a, smem0, bar0, cw, lane, j0, tiles, tile_px, abort_flag);
            } else {
                if (a.pl) pw_stem_builder<2, 1>(a, smem0, bar0, cw, lane, j0, tiles, tile_px, abort_flag);
                else pw_stem_builder<2, 0>(a, smem0, bar0, cw, lane, j0, tiles, tile_px, abort_flag);
            }
        } else if (a.mode != 0) {
            const int cw = warp - 18, ct = tid - 18 * 32;
            int s = 0; uint32_t ph = 0;
            int r = 0; uint32_t rph = 0;
            bool alive = true;
            for (int t = j0; t < tiles && alive; t += a.cpm) {
                for (int ki = 0; ki < k_iters; ++ki) {
                    if (ct == 0) *cp_ok = (ptx::mbar_wait_sleeping(raw_full(r), rph, abort_flag) && ptx::mbar_wait_sleeping(empty(s), ph ^ 1u, abort_flag)) ? 1 : 0;
                    ptx::named_barrier_sync(2, 128);
                    if (!*cp_ok) { alive = false; break; }
                    uint8_t* dst = sStages + (size_t)s * a.stage_bytes;
                    const uint8_t* raw = smem + a.off_raw + (size_t)r * a.raw_bytes;      // [row][HW] as in memory
                    const int c_lo = ki * KC;
                    {
                        // a warp takes two of every eight rows, a lane one 16-byte chunk (four words, the row's start is word
                        // aligned only) of one of the two: four loads, one 16-byte store.  The last chunk of a row runs into the
                        // next row: pixels past HW, which nothing stores.
                        const int ci = lane & 15, nch = (a.HW + 15) >> 4;
                        const uint32_t raw_s = ptx::smem_u32(raw) + (uint32_t)ci * 16u;
                        const uint32_t dst_s = ptx::smem_u32(dst) + ((uint32_t)ci >> 3) * blk_bytes;
                        const uint32_t ci7 = (uint32_t)ci & 7u;
                        if (ci < nch) {
#pragma unroll 2
                            for (int rr = 2 * cw + (lane >> 4); rr < KC; rr += 8) {
                                if (c_lo + rr >= a.C) break;                            // rows past C: zero weights, any finite byte serves
                                const uint32_t src = raw_s + (uint32_t)(rr * a.HW);
                                const uint32_t x0 = lds_u32<0>(src), x1 = lds_u32<4>(src), x2 = lds_u32<8>(src), x3 = lds_u32<12>(src);
                                sts_u128(dst_s + (uint32_t)rr * 128u + ((ci7 ^ ((uint32_t)rr & 7u)) << 4), x0, x1, x2, x3);
                            }
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    ptx::named_barrier_sync(2, 128);
                    if (ct == 0) { ptx::mbar_arrive(full(s)); ptx::mbar_arrive(raw_empty(r)); }
                    if (++s == S) { s = 0; ph ^= 1u; }
                    if (++r == a.raws) { r = 0; rph ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: 16 warps; a TMEM lane quarter (32 filters) is
        // served by four warps that take the tile's 32-pixel chunks in turn
        const int quarter = warp & 3, cg = (warp - 2) >> 2;
        const bool leader = warp == 4 && lane == 0;                   // a thread of quarter 0, which always exists
        const uint32_t n_epi = (uint32_t)live_q * 128u;               // epilogue threads that take part (the others return at once)
        int e = 0;                                                    // index among them: the live warps in ascending order
        for (int wv = 2; wv < warp; ++wv) e += (wv & 3) < live_q ? 32 : 0;
        e += lane;
        const int m_local = quarter * 32 + lane;
        const int grp = a.G > 1 ? m_local / a.m_pad : 0;              // this lane's pixel group (block-diagonal form)
        const int m = a.G > 1 ? m_local - grp * a.m_pad : mt * 128 + m_local;
        const bool live = m < a.M;
        const float mlt = live ? __ldg(a.mult + m) : 1.0f;
        const int bs = live ? __ldg(a.bias + m) : 0;
        const int cp = (live && a.act_mode == 1) ? __ldg(a.cap + m) : 0x7fffffff;
        const Requant rq{a.y_scale, a.y_zp, a.act, a.lut ? sLut : nullptr};
        const uint32_t hi4 = a.act == ZANT_QACT_RELU6 ? 0x01010101u * (uint32_t)(a.six & 255) : 0x7f7f7f7fu;
        const bool quarter_live = quarter < live_q;                   // warps of a quarter whose 32 filters do not exist have nothing to do
        const int rows_here = min(128, a.M - mt * 128);
        int tile_it = 0;
        for (int t = quarter_live ? j0 : tiles; t < tiles; t += a.cpm, ++tile_it) {
            const int b = tile_it & 1;
            const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
            const int img = t / a.px_tiles, p0 = (t - img * a.px_tiles) * tile_px + grp * a.n_px;   // this lane's first pixel
            const int n_valid = min(a.n_px, a.HW - p0);                 // this lane's pixels (all lanes' when G == 1)
            const int n_loop = a.G > 1 ? min(a.n_px, a.HW - (t - img * a.px_tiles) * tile_px) : n_valid;   // warp-uniform chunk bound
            if (a.mode == 0) {
                int ok = 1;
                if (lane == 0) ok = ptx::mbar_wait_sleeping(tfull(b), bph, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            } else {
                // the bulk copy that last read this tile's staging buffer (the previous tile's, or with two buffers the one before) must be through
                if (leader) { if (a.bulk_out) { if (a.outs == 2) ptx::bulk_wait_read<1>(); else ptx::bulk_wait_read<0>(); } *epi_ok = ptx::mbar_wait_sleeping(tfull(b), bph, abort_flag) ? 1 : 0; }
                ptx::named_barrier_sync(1, n_epi);
                if (!*epi_ok) break;
            }
            ptx::tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * 256);
            uint8_t* sOut = sOut0 + ((a.outs == 2 && (tile_it & 1)) ? a.out_stride : 0);
            uint8_t* yrow = a.y + ((size_t)img * a.M + (size_t)m) * a.HW + p0;
            // 16 accumulators -> four packed words
            auto requant16 = [&](const uint32_t (&v)[16], uint32_t* pk) {
                if constexpr (LEAN) {
                    // one (uniform) branch per 16 values, none inside the unrolled loops
                    if (a.act_mode == 1) {
                        // ReLU / ReLU6 as a clamp of the accumulator, fused with the bias add
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4)
                            pk[j4] = pack_sat_s8x4(rq_round(__viaddmin_s32_relu((int)v[j4 * 4 + 0], bs, cp), mlt), rq_round(__viaddmin_s32_relu((int)v[j4 * 4 + 1], bs, cp), mlt),
                                                   rq_round(__viaddmin_s32_relu((int)v[j4 * 4 + 2], bs, cp), mlt), rq_round(__viaddmin_s32_relu((int)v[j4 * 4 + 3], bs, cp), mlt));
                    } else if (a.act_mode == 0) {
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4)
                            pk[j4] = pack_sat_s8x4(rq_round((int)v[j4 * 4 + 0] + bs, mlt), rq_round((int)v[j4 * 4 + 1] + bs, mlt),
                                                   rq_round((int)v[j4 * 4 + 2] + bs, mlt), rq_round((int)v[j4 * 4 + 3] + bs, mlt));
                    } else {
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4)
                            pk[j4] = pack_act_s8x4(rq_round((int)v[j4 * 4 + 0] + bs, mlt), rq_round((int)v[j4 * 4 + 1] + bs, mlt),
                                                   rq_round((int)v[j4 * 4 + 2] + bs, mlt), rq_round((int)v[j4 * 4 + 3] + bs, mlt), true, hi4);
                    }
                } else {
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        uint32_t w4 = 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int acc = (int)v[j4 * 4 + j] + bs;
                            int q = a.out_u8 ? requant_one<true>(acc, mlt, Requant{rq.y_scale, rq.y_zp, rq.act, nullptr})
                                             : requant_one<false>(acc, mlt, Requant{rq.y_scale, rq.y_zp, rq.act, nullptr});
                            if (a.lut) q = (int)sLut[q & 255];
                            w4 |= (uint32_t)(q & 255) << (8 * j);
                        }
                        pk[j4] = w4;
                    }
                }
            };
            // This warp's 32-pixel chunks (cg, cg + 4), each as two halves of 16 columns: the TMEM load of the next half is in
            // flight while the current one is requantised (a wait covers every load issued so far, so a load is issued right
            // after the wait that precedes the arithmetic it overlaps).
            uint32_t va[16], vb[16];
            int ch = cg;
            bool has = ch * 32 < n_loop;
            if (has) ptx::tmem_ld16(taddr + (uint32_t)(ch * 32), va);
            while (has) {
                uint32_t pk[8];
                ptx::tmem_wait_ld();
                ptx::tmem_ld16(taddr + (uint32_t)(ch * 32 + 16), vb);
                requant16(va, pk);
                ptx::tmem_wait_ld();
                const int nch = ch + 4;
                const bool nhas = nch * 32 < n_loop;
                if (nhas) ptx::tmem_ld16(taddr + (uint32_t)(nch * 32), va);
                requant16(vb, pk + 4);
                if (LEAN && a.lut) {
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) pk[j4] = lut4_smem(sLut, pk[j4]);
                }
                const int c0 = ch * 32;
                if (a.mode != 1) {
                    // HW, p0 and c0 are multiples of 16: the chunk's valid part is 16 or 32 bytes
                    if (live && c0 < n_valid) {
                        if (c0 + 32 <= n_valid) {
                            if (a.wide_store) st_global_32B(yrow + c0, pk);
                            else {
                                *reinterpret_cast<uint4*>(yrow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                *reinterpret_cast<uint4*>(yrow + c0 + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                            }
                        } else {
                            *reinterpret_cast<uint4*>(yrow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        }
                    }
                } else {
                    uint32_t* o = reinterpret_cast<uint32_t*>(sOut + (size_t)m_local * a.HW + c0);
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4)
                        if (c0 + j4 * 4 < n_valid) o[j4] = pk[j4];
                }
                ch = nch; has = nhas;
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty(b));
            if (a.mode == 1) {
                // the staged block [rows_here][HW] is the image's contiguous run of these filters' planes
                ptx::fence_proxy_async_smem();
                ptx::named_barrier_sync(1, n_epi);
                uint8_t* dst = a.y + ((size_t)img * a.M + (size_t)mt * 128) * a.HW;
                const int bytes = rows_here * a.HW;
                if (a.bulk_out) {
                    if (leader) bulk_s2g(dst, ptx::smem_u32(sOut), (uint32_t)bytes);
                } else {
                    for (int i = e; i < bytes; i += (int)n_epi) dst[i] = sOut[i];
                    ptx::named_barrier_sync(1, n_epi);
                }
            }
        }
        if (a.mode == 1 && a.bulk_out && leader) bulk_wait_all();
    }

    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, 512);
    if (tid == 0 && *abort_flag) atomicExch(a.status, (int)DEV_ERR_WAIT_TIMEOUT);
}

// =============================================================================================
// Host side
// =============================================================================================
struct PwConvPlan {
    PwConvArgs a{};
    int m_tiles = 0;
    size_t smem_bytes = 0;
    size_t w_bytes = 0;          // blocked weights: [filter tile][k16][128][16]
};

// Chooses the tiling; false when the kernel does not take the shape (the caller falls back to the implicit-GEMM kernel).
inline bool pw_conv_plan(const ConvGeom& g, bool w_zp_all_zero, int sm_count, PwConvPlan& p) {
    if (g.G != 1 || !w_zp_all_zero || g.KH != 1 || g.KW != 1 || g.sh != 1 || g.sw != 1) return false;
    if (g.pt != 0 || g.pl != 0 || g.pb != 0 || g.pr != 0) return false;
    const long long hw = (long long)g.H * g.W;
    if (g.N <= 0 || hw <= 0 || hw > (1 << 24) || g.C > 960 || g.C % 4 != 0) return false;
    if ((long long)g.N * hw < 256) return false;
    PwConvArgs& a = p.a;
    a = PwConvArgs{};
    a.N = g.N; a.C = g.C; a.M = g.M; a.HW = (int)hw;
    a.k_steps = (g.C + 31) / 32;
    a.KS = a.k_steps >= 2 ? 2 : 1;
    a.G = 1; a.m_pad = 128; a.a_steps = a.k_steps;
    p.m_tiles = (g.M + 127) / 128;
    if (p.m_tiles > sm_count) return false;
    if (hw % 16 == 0 && hw >= 128) {
        a.mode = 0;
        // at most 64 filters: G groups of m_pad lanes, each on its own run of pixels (block-diagonal A, G times the K depth),
        // when the deeper A still fits beside the stages
        if (g.M <= 64) {
            const int m_pad = g.M <= 16 ? 16 : (g.M <= 32 ? 32 : 64), G = 128 / m_pad;
            const int steps = G * ((a.k_steps + a.KS - 1) / a.KS) * a.KS;
            if (steps <= 30 && hw >= (long long)G * 64) { a.G = G; a.m_pad = m_pad; a.a_steps = steps; }
        }
        // up to 32 filters fill one lane quarter only (one of the SM's four schedulers would do the whole epilogue): without
        // the groups the pixels-on-lanes form of the implicit-GEMM kernel is the better one
        if (a.G == 1 && g.M <= 32) return false;
        const long long tile_max = 256LL * a.G;
        a.px_tiles = (int)((hw + tile_max - 1) / tile_max);
        a.n_px = (int)(((hw + (long long)a.px_tiles * a.G - 1) / ((long long)a.px_tiles * a.G) + 15) / 16 * 16);
        a.wide_store = (hw % 32 == 0 && a.n_px % 32 == 0) ? 1 : 0;
    } else {
        if (hw > 256 || hw % 4 != 0) return false;      // rows that are not whole words stay with the im2col path (the byte copies cost more than they save)
        a.mode = 1;
        a.px_tiles = 1;
        a.n_px = (int)((hw + 15) / 16 * 16);
        const long long last_rows = g.M - (p.m_tiles - 1) * 128;
        a.bulk_out = (((long long)g.M * hw) % 16 == 0 && (128 * hw) % 16 == 0 && (last_rows * hw) % 16 == 0) ? 1 : 0;
    }
    a.PB = a.n_px > 128 ? 2 : 1;
    const long long tiles = (long long)g.N * a.px_tiles;
    if (tiles > 0x7fffffffLL) return false;
    a.cpm = (int)std::max<long long>(1, std::min<long long>(sm_count / p.m_tiles, tiles));
    a.stage_bytes = a.PB * a.KS * 32 * 128;
    const int a_bytes = a.a_steps * 4096;
    a.out_stride = a.mode == 0 ? 0 : (int)((128 * hw + 1023) / 1024 * 1024);
    a.raw_bytes = a.mode == 0 ? 0 : (int)(((long long)a.KS * 32 * hw + 127) / 128 * 128);
    a.raws = a.mode == 0 ? 0 : 3;
    a.outs = a.mode == 0 ? 0 : 2;
    int budget = 232448 - kPwTail - a_bytes - a.outs * a.out_stride - a.raws * a.raw_bytes;
    if (a.mode != 0 && budget < 4 * a.stage_bytes) { a.outs = 1; budget += a.out_stride; }
    if (a.mode != 0 && budget < 2 * a.stage_bytes) { a.raws = 2; budget += a.raw_bytes; }
    const int out_bytes = a.outs * a.out_stride;
    a.stages = std::min(a.mode == 0 ? kPwMaxStages : 4, budget / a.stage_bytes);
    if (a.stages < 2) return false;
    a.off_stages = a_bytes;                                  // a multiple of 4096: the stages are 1024-byte aligned
    a.off_raw = a.off_stages + a.stages * a.stage_bytes;     // 128-byte aligned (bulk copies want 16)
    a.off_out = a.off_raw + a.raws * a.raw_bytes;
    a.off_tail = (a.off_out + out_bytes + 127) / 128 * 128;
    p.smem_bytes = (size_t)a.off_tail + kPwTail;
    p.w_bytes = (size_t)p.m_tiles * a_bytes;
    return true;
}

// 3x3 stems (at most three input channels, stride 1 or 2, at most 64 filters) on the same kernel: the patches of the input are
// written as the B operand in shared memory (mode 2).  False when the shape is not taken.  The weights ([M][cin][3][3]) go
// through pw_conv_prepare as [M][9 * cin].
inline bool pw_stem_plan(const ConvGeom& g, bool w_zp_all_zero, int x_zp, int sm_count, PwConvPlan& p) {
    if (g.G != 1 || !w_zp_all_zero || g.C > 3 || g.C < 1 || g.KH != 3 || g.KW != 3 || g.dh != 1 || g.dw != 1) return false;
    if (g.sh != g.sw || (g.sh != 1 && g.sh != 2)) return false;
    if (g.pt > 1 || g.pl > 1 || g.pb > 1 || g.pr > 1 || g.pt < 0 || g.pl < 0) return false;
    if (g.M > 64 || g.M < 1 || g.OH <= 0 || g.OW <= 0 || g.N <= 0) return false;
    const long long hw = (long long)g.OH * g.OW;
    // input rows are copied in bulk (16-byte units); the 16 output pixels of a stage chunk lie in one row
    if (g.W % 16 != 0 || g.OW % 16 != 0 || hw % 16 != 0 || hw > (1 << 24) || (long long)g.H * g.W > (1 << 24)) return false;
    // of a word's four input pixels only the first may lie left of the image and only the last right of it
    if ((g.OW - 4) * g.sw + 2 - g.pl + 2 * g.sw >= g.W) return false;
    PwConvArgs& a = p.a;
    a = PwConvArgs{};
    a.mode = 2;
    a.N = g.N; a.C = 9 * g.C; a.M = g.M; a.HW = (int)hw;
    a.cin = g.C; a.ih = g.H; a.iw = g.W; a.oh = g.OH; a.ow = g.OW; a.cs = g.sh; a.pt = g.pt; a.pl = g.pl;
    a.pad_word = 0x01010101u * (uint32_t)(x_zp & 255);
    // p / ow by one multiplication: exact while p * ow < 2^32, p < oh * ow
    if (hw * g.OW >= (1LL << 32)) return false;
    a.ow_magic = (uint32_t)((1ULL << 32) / (uint64_t)g.OW) + 1u;
    a.k_steps = 1; a.KS = 1;
    a.m_pad = g.M <= 16 ? 16 : (g.M <= 32 ? 32 : 64);
    a.G = 128 / a.m_pad;
    a.a_steps = a.G;
    p.m_tiles = 1;
    if (hw < (long long)a.G * 64 || (long long)g.N * hw < 4096) return false;
    const long long tile_max = 256LL * a.G;
    a.px_tiles = (int)((hw + tile_max - 1) / tile_max);
    a.n_px = (int)(((hw + (long long)a.px_tiles * a.G - 1) / ((long long)a.px_tiles * a.G) + 15) / 16 * 16);
    a.wide_store = (hw % 32 == 0 && a.n_px % 32 == 0) ? 1 : 0;
    a.PB = a.n_px > 128 ? 2 : 1;
    const long long tiles = (long long)g.N * a.px_tiles;
    if (tiles > 0x7fffffffLL) return false;
    a.cpm = (int)std::max<long long>(1, std::min<long long>(sm_count, tiles));
    a.stage_bytes = a.PB * 4096;
    const long long tile_px = (long long)a.G * a.n_px;
    const long long rows_out = (tile_px + g.OW - 2) / g.OW + 1;             // output rows a tile can touch
    a.band = (int)((rows_out - 1) * a.cs + 3);
    const long long raw = 16 + (long long)a.cin * a.band * a.iw + 16;       // the words in front of the first and behind the last row are read
    if (raw > 40000) return false;
    a.raw_bytes = (int)((raw + 127) / 128 * 128);
    a.raws = 3;                                                             // with two groups per tile the four builder warps work on two tiles

    const int a_bytes = a.a_steps * 4096;
    a.stages = 8;                                                           // builder warp w owns the stages w and w + 4
    a.off_stages = a_bytes;
    a.off_raw = a.off_stages + a.stages * a.stage_bytes;
    a.off_out = a.off_raw + a.raws * a.raw_bytes;
    a.off_tail = (a.off_out + 127) / 128 * 128;
    p.smem_bytes = (size_t)a.off_tail + kPwTail;
    if (p.smem_bytes > 232448) return false;
    p.w_bytes = (size_t)a_bytes;
    return true;
}

// Blocks `w` ([M][C] int8) as [filter tile][k16][128][16] (zero beyond M and C) and folds the input zero point into the bias.
inline void pw_conv_prepare(const PwConvPlan& p, const int8_t* w, const int32_t* bias, int x_zp, std::vector<int8_t>& w_blk, std::vector<int32_t>& bias_f) {
    const PwConvArgs& a = p.a;
    w_blk.assign(p.w_bytes, 0);
    bias_f.assign(a.M, 0);
    const size_t tile_bytes = (size_t)a.a_steps * 4096;
    const int group_steps = a.a_steps / a.G;                  // K steps per pixel group (whole stages)
    for (int m = 0; m < a.M; ++m) {
        long long sum = 0;
        for (int c = 0; c < a.C; ++c) {
            const int8_t v = w[(size_t)m * a.C + c];
            if (a.G == 1) {
                w_blk[(size_t)(m / 128) * tile_bytes + (size_t)(c / 16) * 2048 + (size_t)(m % 128) * 16 + (c % 16)] = v;
            } else {
                // block-diagonal: lane g * m_pad + m, K index g * (group_steps * 32) + c
                for (int gq = 0; gq < a.G; ++gq) {
                    const int k = gq * group_steps * 32 + c, row = gq * a.m_pad + m;
                    w_blk[(size_t)(k / 16) * 2048 + (size_t)row * 16 + (k % 16)] = v;
                }
            }
            sum += v;
        }
        bias_f[m] = (int32_t)((bias ? bias[m] : 0) - (long long)x_zp * sum);
    }
}

template <bool XU8, bool LEAN>
inline int32_t pw_conv_launch_t(zant_ctx* ctx, const PwConvPlan& p, const PwConvArgs& a, const CUtensorMap& x_map, int grid) {
    ZB_SMEM_ATTR(ctx, (tc_pw_nchw_kernel<XU8, LEAN>), 232448);
    tc_pw_nchw_kernel<XU8, LEAN><<<grid, kPwThreads, p.smem_bytes, ctx->stream>>>(a, x_map);
    return check_launch(ctx, "tc_pw_nchw_kernel");
}

// Tensor map over the NCHW input in 4-byte elements, (HW / 4, C, N); box = 128 pixels x a stage's channels, 128-byte swizzle.
// Channels past C and pixels past HW read as zero.
inline int32_t pw_conv_encode_map(const PwConvArgs& a, const void* x, CUtensorMap* map) {
    const cuuint64_t HW = (cuuint64_t)a.HW, C = (cuuint64_t)a.C, N = (cuuint64_t)a.N;
    const cuuint64_t dims[3] = {HW / 4, C, N}, strides[2] = {HW, C * HW};
    const cuuint32_t box[3] = {32, (cuuint32_t)(a.KS * 32), 1}, estr[3] = {1, 1, 1};
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            cudaGetLastError();
            return fail(ZANT_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ZANT_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return ZANT_OK;
}

// Buffers the kernel takes: x 16-byte aligned (tensor map, word loads), y 32-byte aligned (32-byte stores, bulk copies).
inline bool pw_conv_ptr_ok(const void* x, const void* y) {
    return (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(y) & 31u) == 0;
}

// `cap_dev`: per-filter accumulator bounds from requant_relu_caps when that returned true, else null.
inline int32_t pw_conv_run(zant_ctx* ctx, const PwConvPlan& p, const void* x, bool x_u8, const int8_t* w_blk_dev, const float* mult_dev,
                           const int32_t* bias_dev, void* y, bool y_u8, const Requant& rq, bool mult_finite, const int32_t* cap_dev) {
    PwConvArgs a = p.a;
    a.x = (const uint8_t*)x; a.y = (uint8_t*)y; a.w = w_blk_dev; a.mult = mult_dev; a.bias = bias_dev;
    a.y_scale = rq.y_scale; a.y_zp = rq.y_zp; a.act = rq.act; a.out_u8 = y_u8 ? 1 : 0; a.lut = rq.lut;
    const bool lean = !y_u8 && rq.y_zp == 0 && mult_finite;
    if (lean) a.six = lean_six(rq.y_scale);
    a.cap = cap_dev;
    a.act_mode = rq.act == ZANT_QACT_NONE ? 0 : (cap_dev ? 1 : 2);
    a.status = ctx->status_word;
    const int grid = p.m_tiles * a.cpm;
    alignas(64) CUtensorMap x_map{};
    if (a.mode == 0) ZB_TRY(pw_conv_encode_map(a, x, &x_map));
    if (x_u8) return lean ? pw_conv_launch_t<true, true>(ctx, p, a, x_map, grid) : pw_conv_launch_t<true, false>(ctx, p, a, x_map, grid);
    return lean ? pw_conv_launch_t<false, true>(ctx, p, a, x_map, grid) : pw_conv_launch_t<false, false>(ctx, p, a, x_map, grid);
}

}  // namespace zb
