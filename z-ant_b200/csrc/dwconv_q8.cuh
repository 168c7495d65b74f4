// Depthwise 3x3 QLinearConv (group == channels == filters, pads 1, dilation 1, stride 1 or 2) on
// NCHW int8/uint8: an HBM-bound kernel, one pass over the input and one over the output.
//
// A lane owns a strip of a plane: 4 output columns, all rows.  It walks down the input rows with one
// aligned 4-byte load per row (stride 2: two loads, 8 input columns); the neighbouring columns come
// from the adjacent lanes by shuffle.  For each input row it forms the four 3-pixel windows with prmt and
// feeds them to dp4a against the three filter rows (the fourth dp4a weight is 0), accumulating into
// the output rows the input row belongs to; an output row is requantised, packed and stored as one
// 4-byte word once its last input row has been seen.  Several narrow planes share a warp (LW lanes per
// plane).  Pixels outside the image hold the input zero point, which is folded into the bias
// (bias - x_zp * sum(w)) exactly as in the tensor-core paths.
// ALIGNED: rows are whole 4-byte words (W % 4 == 0 and OW % 4 == 0).  Otherwise the four bytes of a lane
// are cut out of the two aligned words that hold them and the outputs are stored bytewise, which covers
// any width (the 14x14 and 7x7 planes of mobile networks).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>
#include <vector>

#include "context.cuh"
#include "geometry.hpp"
#include "fused_cnn.cuh"
#include "kernels_q8.cuh"
#include "ptx_sm100.cuh"

namespace zb {

struct QDwArgs {
    const uint8_t* x; uint8_t* y;
    const uint32_t* wrow;      // [C][3] filter rows packed for dp4a: bytes (w[kh][0], w[kh][1], w[kh][2], 0)
    const float* mult; const int32_t* bias;   // [C]; bias already holds -x_zp * sum(w)
    int planes, C, H, W, OH, OW;
    long long x_bytes;         // size of x (the unaligned variant never reads a word that extends past it)
    int log2LW;                // lanes per plane = 1 << log2LW (covers OW / 4 columns of 4 outputs)
    uint32_t pad_word;
    float y_scale; int y_zp; int act; int out_u8;
    const uint8_t* lut;       // optional table applied to the output codes (see Requant)
    int six;
    const int32_t* cap;       // lean epilogue, act_mode 1: per-channel accumulator bound of the activation (requant_relu_caps)
    int act_mode;             // lean epilogue: 0 no activation, 1 clamp of the accumulator to [0, cap], 2 clamp of the packed codes
};

template <bool XU8>
__device__ __forceinline__ int dw_dp4a(uint32_t x, uint32_t w, int acc) {
    int d;
    if (XU8) asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(acc));
    else asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(acc));
    return d;
}

// Requantises four accumulators of one channel and packs them (little endian = ascending columns).
// `cp`: the channel's accumulator bound (act_mode 1).  ACC: the kernel takes the accumulator form of the activation (measured
// faster in the row-sliding kernel, slower in the 8-column and flat ones, which keep the clamp of the packed codes).
template <bool LEAN, bool ACC = true>
__device__ __forceinline__ uint32_t dw_requant4(const int acc[4], float m, int cp, const QDwArgs& p) {
    if (LEAN) {
        uint32_t pk;
        if (ACC && p.act_mode == 1) {
            // ReLU / ReLU6 as a clamp of the accumulator: one instruction per value
            pk = pack_sat_s8x4(rq_round(__viaddmin_s32_relu(acc[0], 0, cp), m), rq_round(__viaddmin_s32_relu(acc[1], 0, cp), m),
                               rq_round(__viaddmin_s32_relu(acc[2], 0, cp), m), rq_round(__viaddmin_s32_relu(acc[3], 0, cp), m));
        } else {
            pk = pack_act_s8x4(rq_round(acc[0], m), rq_round(acc[1], m), rq_round(acc[2], m), rq_round(acc[3], m), p.act != ZANT_QACT_NONE,
                               p.act == ZANT_QACT_RELU6 ? 0x01010101u * (uint32_t)(p.six & 255) : 0x7f7f7f7fu);
        }
        if (p.lut) pk = lut4(p.lut, pk);
        return pk;
    }
    const Requant rq{p.y_scale, p.y_zp, p.act, p.lut};
    uint32_t pk = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q = p.out_u8 ? requant_one<true>(acc[i], m, rq) : requant_one<false>(acc[i], m, rq);
        pk |= (uint32_t)(q & 255) << (8 * i);
    }
    return pk;
}

// STRIDE 1: lane = 4 input columns = 4 output columns.  STRIDE 2: lane = 8 input columns = 4 output columns.
// Four consecutive bytes of x starting at byte offset `off` (any alignment); bytes at or beyond `limit`
// (the end of the row) are replaced by the padding byte.
__device__ __forceinline__ uint32_t dw_load_unaligned(const QDwArgs& p, long long off, int n_valid) {
    uint32_t v;
    if (off + 8 <= p.x_bytes) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(p.x) + (off >> 2);
        const uint32_t a = __ldg(w), b = __ldg(w + 1);
        v = __byte_perm(a, b, 0x3210u + 0x1111u * (uint32_t)(off & 3));
    } else {                   // the last bytes of the tensor: one by one
        v = 0;
        for (int i = 0; i < 4; ++i)
            if (off + i < p.x_bytes) v |= (uint32_t)__ldg(p.x + off + i) << (8 * i);
    }
    if (n_valid < 4) {
        const uint32_t mask = n_valid <= 0 ? 0u : (0xffffffffu >> (8 * (4 - n_valid)));
        v = (v & mask) | (p.pad_word & ~mask);
    }
    return v;
}

// SMEM: for planes whose rows are not whole words (W % 4 != 0: 14 x 14, 7 x 7, odd sizes).  The CTA's planes (8 warps x
// planes per warp, consecutive in memory) are first copied into shared memory with rows padded to whole 8-byte groups
// (pad bytes = the input zero point), the sliding-row arithmetic then reads aligned words from there and writes its
// packed output words into a padded output image in shared memory, and a last phase copies the output rows out.  Global
// memory is touched by row-wise byte copies of consecutive rows only; the arithmetic is that of the aligned form.
// SIN: the input planes are staged too; false with SMEM = true is the form for input rows of whole words (aligned loads
// straight from global memory) whose OUTPUT rows are not (stride 2 from 28 x 28 to 14 x 14): only the output is staged.
template <int STRIDE, bool XU8, bool LEAN, bool ALIGNED, bool SMEM = false, bool SIN = SMEM>
__global__ void __launch_bounds__(256) qdwconv3x3_kernel(const QDwArgs p) {
    extern __shared__ __align__(16) uint8_t dw_smem[];
    const int lane = threadIdx.x & 31;
    const int LW = 1 << p.log2LW;
    const int ppw = 32 >> p.log2LW;                          // planes per warp
    const int sub = lane >> p.log2LW, col = lane & (LW - 1);
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int groups = (p.planes + ppw - 1) / ppw;
    const int Wp = SIN ? (p.W + 7) / 8 * 8 : p.W;            // padded row pitches of the shared-memory images
    const int OWp = SMEM ? (p.OW + 3) / 4 * 4 : p.OW;
    const int in_words = SIN ? Wp >> 2 : p.W >> 2;           // 4-byte words per input row
    const bool col_ok = col * 4 < p.OW;
    const int out_valid = p.OW - col * 4;                    // output columns of this lane (>= 4: all)
    const int wib = threadIdx.x >> 5;                        // warp in block
    const int P = 8 * ppw;                                   // planes per CTA pass (SMEM)
    uint8_t* const s_in = dw_smem;
    uint8_t* const s_out = dw_smem + (SIN ? (size_t)P * p.H * Wp : 0);
    const int g_first = SMEM ? (int)blockIdx.x * 8 + wib : (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int g_step = SMEM ? (int)gridDim.x * 8 : warps;
    for (int g = g_first; SMEM ? (g - wib < groups) : (g < groups); g += g_step) {
        const int plane = g * ppw + sub;
        const bool live = plane < p.planes && col_ok;
        if (SMEM && !SIN) __syncthreads();                       // the previous pass's copy-out has left the output image
        if (SIN) {
            // phase 1: the pass's planes are one contiguous run of bytes in global memory (it starts at a multiple of
            // 8 planes, hence at a word boundary): consecutive threads load consecutive words and scatter their bytes
            // into the padded image.  The pad columns are written once, before the first pass.
            const int plane0 = (g - wib) * ppw;
            const int n_pl = min(P, p.planes - plane0);
            const int n_bytes = n_pl * p.H * p.W;
            const uint8_t* src = p.x + (size_t)plane0 * p.H * p.W;
            if (g == g_first) {
                for (int rr = threadIdx.x; rr < P * p.H; rr += 256)
                    for (int i = p.W; i < Wp; ++i) s_in[(size_t)rr * Wp + i] = (uint8_t)p.pad_word;
            }
            for (int w = threadIdx.x; w * 4 < n_bytes; w += 256) {
                const int b0 = w * 4;
                uint32_t v;
                if (b0 + 4 <= n_bytes) v = __ldg(reinterpret_cast<const uint32_t*>(src) + w);
                else { v = 0; for (int i = 0; b0 + i < n_bytes; ++i) v |= (uint32_t)__ldg(src + b0 + i) << (8 * i); }
                int row = b0 / p.W, iw = b0 - row * p.W;            // row counts the rows of all planes of the pass
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (b0 + i < n_bytes) s_in[(size_t)row * Wp + iw] = (uint8_t)(v >> (8 * i));
                    if (++iw == p.W) { iw = 0; ++row; }
                }
            }
            __syncthreads();
        }
        const int c = live ? plane % p.C : 0;
        const uint32_t k0 = __ldg(p.wrow + c * 3), k1 = __ldg(p.wrow + c * 3 + 1), k2 = __ldg(p.wrow + c * 3 + 2);
        const float m = __ldg(p.mult + c);
        const int b = __ldg(p.bias + c);
        const int cp = p.act_mode == 1 ? __ldg(p.cap + c) : 0x7fffffff;
        const int pl_local = wib * ppw + sub;                 // SMEM: this lane's plane within the pass
        const uint32_t* xin = SIN ? reinterpret_cast<const uint32_t*>(s_in + (size_t)pl_local * p.H * Wp)
                                   : reinterpret_cast<const uint32_t*>(p.x + (size_t)(live ? plane : 0) * p.H * p.W);
        uint32_t* yout = SMEM ? reinterpret_cast<uint32_t*>(s_out + (size_t)pl_local * p.OH * OWp) + col
                              : reinterpret_cast<uint32_t*>(p.y + (size_t)(live ? plane : 0) * p.OH * p.OW) + col;
        const int ow_words = SMEM ? OWp >> 2 : p.OW >> 2;
        const long long xplane = (long long)(live ? plane : 0) * p.H * p.W;
        uint8_t* yplane = p.y + (size_t)(live ? plane : 0) * p.OH * p.OW + col * 4;
        auto store_row = [&](int oh, uint32_t pk) {
            if (!live) return;
            if (ALIGNED || SMEM) { yout[(size_t)oh * ow_words] = pk; return; }
            uint8_t* d = yplane + (size_t)oh * p.OW;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < out_valid) d[i] = (uint8_t)(pk >> (8 * i));
        };

        if (STRIDE == 1) {
            // acc[r]: output row (ih - 1 + r) while input row ih is being added; rows rotate through the three slots
            int acc[3][4];
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[r][i] = b;
            // input rows -1 .. H (the first and last are padding), three per trip; the loads of the next trip
            // are issued before this trip's arithmetic so that their latency is covered
            auto load_row = [&](int ih) -> uint32_t {
                if (!(live && ih >= 0 && ih < p.H)) return p.pad_word;
                if (SIN) return xin[ih * in_words + col];
                if (ALIGNED) return __ldg(xin + (size_t)ih * in_words + col);
                return dw_load_unaligned(p, xplane + (long long)ih * p.W + col * 4, p.W - col * 4);
            };
            uint32_t nx0 = load_row(-1), nx1 = load_row(0), nx2 = load_row(1);
            for (int base = -1; base <= p.H; base += 3) {
                const uint32_t cur_rows[3] = {nx0, nx1, nx2};
                nx0 = load_row(base + 3); nx1 = load_row(base + 4); nx2 = load_row(base + 5);
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    const int ih = base + r;
                    if (ih > p.H) break;
                    const uint32_t M = cur_rows[r];
                    uint32_t L = __shfl_up_sync(0xffffffffu, M, 1), R = __shfl_down_sync(0xffffffffu, M, 1);
                    if (col == 0) L = p.pad_word;
                    if (col * 4 + 4 >= p.W) R = p.pad_word;
                    const uint32_t w0 = __byte_perm(L, M, 0x6543), w1 = M, w2 = __byte_perm(M, R, 0x4321), w3 = __byte_perm(M, R, 0x5432);
                    // base is -1 mod 3, so r is (ih + 1) % 3 at compile time and names the slots of the three output rows
                    int* a_prev = acc[(r + 2) % 3];   // output row ih - 1: this input row is its filter row 2
                    int* a_cur = acc[r % 3];          // output row ih: filter row 1
                    int* a_next = acc[(r + 1) % 3];   // output row ih + 1: filter row 0
                    a_prev[0] = dw_dp4a<XU8>(w0, k2, a_prev[0]); a_prev[1] = dw_dp4a<XU8>(w1, k2, a_prev[1]);
                    a_prev[2] = dw_dp4a<XU8>(w2, k2, a_prev[2]); a_prev[3] = dw_dp4a<XU8>(w3, k2, a_prev[3]);
                    a_cur[0] = dw_dp4a<XU8>(w0, k1, a_cur[0]); a_cur[1] = dw_dp4a<XU8>(w1, k1, a_cur[1]);
                    a_cur[2] = dw_dp4a<XU8>(w2, k1, a_cur[2]); a_cur[3] = dw_dp4a<XU8>(w3, k1, a_cur[3]);
                    a_next[0] = dw_dp4a<XU8>(w0, k0, a_next[0]); a_next[1] = dw_dp4a<XU8>(w1, k0, a_next[1]);
                    a_next[2] = dw_dp4a<XU8>(w2, k0, a_next[2]); a_next[3] = dw_dp4a<XU8>(w3, k0, a_next[3]);
                    // output row ih - 1 has now seen its three input rows
                    const int oh = ih - 1;
                    if (oh >= 0 && oh < p.OH) {
                        store_row(oh, dw_requant4<LEAN>(a_prev, m, cp, p));
                    }
                    a_prev[0] = a_prev[1] = a_prev[2] = a_prev[3] = b;   // the slot becomes output row ih + 2
                }
            }
        } else {
            // stride 2: output row oh reads input rows 2oh-1, 2oh, 2oh+1; lane holds input columns 8col .. 8col+7
            int nxt[4] = {b, b, b, b};      // output row oh+1 so far (its filter row 0 = input row 2oh+1)
            const bool c0 = live && col * 8 < p.W, c1 = live && col * 8 + 4 < p.W;
            auto load_w = [&](int ih, int k, bool on) -> uint32_t {
                if (!(on && ih < p.H)) return p.pad_word;
                if (SIN) return xin[ih * in_words + col * 2 + k];
                if (ALIGNED) return __ldg(xin + (size_t)ih * in_words + col * 2 + k);
                return dw_load_unaligned(p, xplane + (long long)ih * p.W + col * 8 + k * 4, p.W - col * 8 - k * 4);
            };
            // the four words of the next output row are loaded while this one is computed
            uint32_t n00 = load_w(0, 0, c0), n01 = load_w(0, 1, c1), n10 = load_w(1, 0, c0), n11 = load_w(1, 1, c1);
            for (int oh = 0; oh < p.OH; ++oh) {
                int cur[4] = {nxt[0], nxt[1], nxt[2], nxt[3]};
#pragma unroll
                for (int i = 0; i < 4; ++i) nxt[i] = b;
                if (oh == 0) {
                    // input row -1 is padding: filter row 0 sees the zero point everywhere
#pragma unroll
                    for (int i = 0; i < 4; ++i) cur[i] = dw_dp4a<XU8>(p.pad_word, k0, cur[i]);
                }
                const uint32_t rows[2][2] = {{n00, n01}, {n10, n11}};
                n00 = load_w(2 * oh + 2, 0, c0); n01 = load_w(2 * oh + 2, 1, c1);
                n10 = load_w(2 * oh + 3, 0, c0); n11 = load_w(2 * oh + 3, 1, c1);
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const uint32_t M0 = rows[rr][0], M1 = rows[rr][1];
                    uint32_t L = __shfl_up_sync(0xffffffffu, M1, 1);
                    if (col == 0) L = p.pad_word;
                    // windows centred on input columns 8col, 8col+2, 8col+4, 8col+6
                    const uint32_t w0 = __byte_perm(L, M0, 0x6543), w1 = __byte_perm(M0, M0, 0x0321);
                    const uint32_t w2 = __byte_perm(M0, M1, 0x6543), w3 = __byte_perm(M1, M1, 0x0321);
                    if (rr == 0) {          // input row 2oh: filter row 1 of this output row
                        cur[0] = dw_dp4a<XU8>(w0, k1, cur[0]); cur[1] = dw_dp4a<XU8>(w1, k1, cur[1]);
                        cur[2] = dw_dp4a<XU8>(w2, k1, cur[2]); cur[3] = dw_dp4a<XU8>(w3, k1, cur[3]);
                    } else {                // input row 2oh+1: filter row 2 of this output row, filter row 0 of the next
                        cur[0] = dw_dp4a<XU8>(w0, k2, cur[0]); cur[1] = dw_dp4a<XU8>(w1, k2, cur[1]);
                        cur[2] = dw_dp4a<XU8>(w2, k2, cur[2]); cur[3] = dw_dp4a<XU8>(w3, k2, cur[3]);
                        nxt[0] = dw_dp4a<XU8>(w0, k0, nxt[0]); nxt[1] = dw_dp4a<XU8>(w1, k0, nxt[1]);
                        nxt[2] = dw_dp4a<XU8>(w2, k0, nxt[2]); nxt[3] = dw_dp4a<XU8>(w3, k0, nxt[3]);
                    }
                }
                store_row(oh, dw_requant4<LEAN>(cur, m, cp, p));
            }
        }
        if (SMEM) {
            // phase 3: the pass's outputs are one contiguous run too: consecutive threads gather four bytes from the
            // padded image and store consecutive words
            __syncthreads();
            const int plane0 = (g - wib) * ppw;
            const int n_pl = min(P, p.planes - plane0);
            const int n_bytes = n_pl * p.OH * p.OW;
            uint8_t* dst = p.y + (size_t)plane0 * p.OH * p.OW;
            for (int w = threadIdx.x; w * 4 < n_bytes; w += 256) {
                const int b0 = w * 4;
                int row = b0 / p.OW, ow = b0 - row * p.OW;
                uint32_t v = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (b0 + i < n_bytes) v |= (uint32_t)s_out[(size_t)row * OWp + ow] << (8 * i);
                    if (++ow == p.OW) { ow = 0; ++row; }
                }
                if (b0 + 4 <= n_bytes) reinterpret_cast<uint32_t*>(dst)[w] = v;
                else for (int i = 0; b0 + i < n_bytes; ++i) dst[b0 + i] = (uint8_t)(v >> (8 * i));
            }
        }
    }
}

// Stride 1 on planes whose rows are whole 8-byte groups (W % 8 == 0): a lane owns 8 columns (one 8-byte
// load per row), which halves the per-output share of loads, shuffles and address arithmetic; the padding
// rows and the first output row are peeled off so that the row loop carries no range checks.
template <bool XU8, bool LEAN>
__global__ void __launch_bounds__(256) qdwconv3x3_s1w8_kernel(const QDwArgs p) {
    const int lane = threadIdx.x & 31;
    const int LW = 1 << p.log2LW;                            // lanes per plane, each 8 columns
    const int ppw = 32 >> p.log2LW;
    const int sub = lane >> p.log2LW, col = lane & (LW - 1);
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int groups = (p.planes + ppw - 1) / ppw;
    const int wu2 = p.W >> 3;                                // 8-byte groups per row
    const bool col_ok = col < wu2;
    const bool first_col = col == 0, last_col = col == wu2 - 1;
    const uint2 padrow = make_uint2(p.pad_word, p.pad_word);
    for (int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < groups; g += warps) {
        const int plane = g * ppw + sub;
        const bool live = plane < p.planes && col_ok;
        const int c = live ? plane % p.C : 0;
        const uint32_t k0 = __ldg(p.wrow + c * 3), k1 = __ldg(p.wrow + c * 3 + 1), k2 = __ldg(p.wrow + c * 3 + 2);
        const float m = __ldg(p.mult + c);
        const int b = __ldg(p.bias + c);
        const uint2* xr = reinterpret_cast<const uint2*>(p.x + (size_t)(live ? plane : 0) * p.H * p.W) + (live ? col : 0);
        uint2* yr = reinterpret_cast<uint2*>(p.y + (size_t)(live ? plane : 0) * p.H * p.W) + (live ? col : 0);
        int A[8], B[8], C[8];                                // three output rows in flight
#pragma unroll
        for (int i = 0; i < 8; ++i) A[i] = B[i] = C[i] = b;
        // adds input row M to the output rows above (filter row 2), at (1) and below (0) it
        auto step = [&](const uint2 M, int* up, int* at, int* dn) {
            uint32_t L = __shfl_up_sync(0xffffffffu, M.y, 1), R = __shfl_down_sync(0xffffffffu, M.x, 1);
            if (first_col) L = p.pad_word;
            if (last_col) R = p.pad_word;
            const uint32_t w[8] = {__byte_perm(L, M.x, 0x6543), M.x, __byte_perm(M.x, M.y, 0x4321), __byte_perm(M.x, M.y, 0x5432),
                                   __byte_perm(M.x, M.y, 0x6543), M.y, __byte_perm(M.y, R, 0x4321), __byte_perm(M.y, R, 0x5432)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (up) up[i] = dw_dp4a<XU8>(w[i], k2, up[i]);
                if (at) at[i] = dw_dp4a<XU8>(w[i], k1, at[i]);
                if (dn) dn[i] = dw_dp4a<XU8>(w[i], k0, dn[i]);
            }
        };
        auto emit = [&](int* row) {                          // requantise, store, and recycle the slot
            const uint2 pk = make_uint2(dw_requant4<LEAN, false>(row, m, 0, p), dw_requant4<LEAN, false>(row + 4, m, 0, p));
            if (live) *yr = pk;
            yr += wu2;
#pragma unroll
            for (int i = 0; i < 8; ++i) row[i] = b;
        };
        auto load = [&]() -> uint2 { const uint2 v = live ? __ldg(xr) : padrow; xr += wu2; return v; };
        // rows -1 (padding) and 0: nothing to emit yet.  A = output row 0, B = row 1, C = row 2.
        step(padrow, nullptr, nullptr, A);
        step(load(), nullptr, A, B);
        int ih = 1;
        // three input rows per trip (the slots return to their roles); the next trip's rows are requested before this
        // trip's arithmetic, so that their latency is covered by it
        uint2 n0 = padrow, n1 = padrow, n2 = padrow;
        if (ih + 2 < p.H) { n0 = load(); n1 = load(); n2 = load(); }
        for (; ih + 2 < p.H; ih += 3) {
            const uint2 r0 = n0, r1 = n1, r2 = n2;
            if (ih + 5 < p.H) { n0 = load(); n1 = load(); n2 = load(); }
            step(r0, A, B, C); emit(A);                      // A becomes output row ih + 2
            step(r1, B, C, A); emit(B);
            step(r2, C, A, B); emit(C);
        }
        // up to two more input rows, then the padding row below the image
        int left = p.H - ih;                                 // 0, 1 or 2 rows (H >= 1)
        if (left == 2) {
            const uint2 r0 = load(), r1 = load();
            step(r0, A, B, C); emit(A);
            step(r1, B, C, nullptr); emit(B);
            step(padrow, C, nullptr, nullptr); emit(C);
        } else if (left == 1) {
            const uint2 r0 = load();
            step(r0, A, B, nullptr); emit(A);
            step(padrow, B, nullptr, nullptr); emit(B);
        } else if (p.H >= 1) {
            step(padrow, A, nullptr, nullptr); emit(A);
        }
    }
}

// Small planes, "rows" form: stride 1 on 14 x 14 and 7 x 7, stride 2 from 28 x 28 and 14 x 14 (W and the stride S are template
// parameters; OW = W for stride 1, W / 2 for stride 2).  A CTA takes batches of PB whole planes,
// which are one run of bytes in NCHW: one bulk copy brings a batch into shared memory, one takes the results back, so every
// global access is a full line however the rows lie.  A thread owns one output row of one plane: per filter row it reads the
// W + 2 bytes col -1 .. col W of the input row as NA + 1 aligned shared-memory words, shifts them to the row's alignment,
// puts the zero point in the two border bytes, and cuts the OW three-byte windows (S bytes apart) out of the NA words (a window
// that starts on a word needs no permute; the dp4a weight of the fourth byte is 0).  The OW results are requantised four at a time and
// stored to the output batch bytewise (two bytes at a time when the rows are 2-byte aligned).  Three input and two output
// buffers: the next two batches are in flight and the previous one is being written back while a batch is computed.
// PB * H * W and PB * OH * OW are multiples of 16 (bulk copies), and a trailing batch of fewer planes is copied by the threads.
struct QDwRowsArgs {
    QDwArgs p;
    int PB;                    // planes per batch
    int batches;               // ceil(planes / PB)
    int buf_bytes;             // PB * H * W
    int out_bytes;             // PB * OH * OW
    int* status;               // device status word: DEV_ERR_WAIT_TIMEOUT when a bounded wait gave up
};

template <bool XU8, bool LEAN, int W, int S>
__global__ void __launch_bounds__(256) qdwconv3x3_rows_kernel(const QDwRowsArgs a) {
    constexpr int NA = (W + 2 + 3) / 4;                             // words that hold the bytes col -1 .. col W
    constexpr int OW = S == 1 ? W : W / 2;
    extern __shared__ __align__(128) uint8_t dw_rows_smem[];
    const QDwArgs& p = a.p;
    const int P = p.H * W, PO = p.OH * OW;
    // [in 0][in 1][in 2][out 0][out 1][barriers]; an input buffer has 16 bytes in front (the word before the first row is read)
    const int in_stride = (a.buf_bytes + 16 + 16 + 127) / 128 * 128, out_stride = (a.out_bytes + 127) / 128 * 128;
    uint8_t* s_in = dw_rows_smem;
    uint8_t* s_out = dw_rows_smem + 3 * in_stride;
    uint64_t* bars = reinterpret_cast<uint64_t*>(dw_rows_smem + 3 * in_stride + 2 * out_stride);
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const int t = threadIdx.x;
    const int pl = t / p.OH, r = t - pl * p.OH;                     // plane of the batch, output row
    const bool worker = pl < a.PB;
    if (t == 0) {
        for (int i = 0; i < 3; ++i) ptx::mbar_init(ptx::smem_u32(&bars[i]), 1);
        abort_flag_s = 0;
        ptx::mbar_fence_init();
    }
    __syncthreads();
    auto planes_of = [&](int b) { return min(a.PB, p.planes - b * a.PB); };
    auto issue_load = [&](int b, int buf) {
        // whole batches by one bulk copy; a trailing partial batch is copied by the threads at its turn
        if (planes_of(b) == a.PB) {
            const uint32_t bar = ptx::smem_u32(&bars[buf]);
            ptx::mbar_arrive_expect_tx(bar, (uint32_t)a.buf_bytes);
            ptx::bulk_g2s(ptx::smem_u32(s_in + buf * in_stride + 16), p.x + (size_t)b * a.buf_bytes, (uint32_t)a.buf_bytes, bar);
        }
    };
    int it = 0;
    if (t == 0) {
        if ((int)blockIdx.x < a.batches) issue_load((int)blockIdx.x, 0);
        if ((int)(blockIdx.x + gridDim.x) < a.batches) issue_load((int)(blockIdx.x + gridDim.x), 1);
    }
    int ibuf = 0;                                                   // input buffer of this batch: it % 3
    // channel of this thread's plane: (b * PB + pl) mod C, kept up to date by adding the grid's stride mod C
    int c = (int)(((long long)blockIdx.x * a.PB + pl) % p.C);
    const int c_step = (int)(((long long)gridDim.x * a.PB) % p.C);
    uint32_t phases = 0;                                            // bit b: phase of barrier b
    for (int b = (int)blockIdx.x; b < a.batches; b += (int)gridDim.x, ++it) {
        const int buf = it & 1;
        const int nb = b + 2 * (int)gridDim.x, nbuf = ibuf == 0 ? 2 : ibuf - 1;       // (it + 2) % 3
        const int n_pl = planes_of(b);
        const bool whole = n_pl == a.PB;
        if (t == 0) {
            ptx::bulk_wait_read<1>();                               // the write-back that read s_out[buf] two batches ago
            if (nb < a.batches) issue_load(nb, nbuf);               // that buffer was last read before the barrier that ended the previous batch
            // one thread waits for this batch's bytes; the barrier below hands them to the others
            if (whole && !ptx::mbar_wait(ptx::smem_u32(&bars[0]) + 8u * (uint32_t)ibuf, (phases >> ibuf) & 1u, abort_flag)) *abort_flag = 1;
        }
        if (whole) phases ^= 1u << ibuf;
        uint8_t* in = s_in + ibuf * in_stride + 16;
        uint8_t* out = s_out + buf * out_stride;
        if (!whole) {
            const uint8_t* src = p.x + (size_t)b * a.buf_bytes;
            for (int i = t; i < n_pl * P; i += 256) in[i] = __ldg(src + i);
        }
        __syncthreads();
        if (*abort_flag) break;
        if (worker && pl < n_pl) {
            const float m = __ldg(p.mult + c);
            const int bs = __ldg(p.bias + c);
            const int cp = p.act_mode == 1 ? __ldg(p.cap + c) : 0x7fffffff;
            int acc[(OW + 3) / 4 * 4];
#pragma unroll
            for (int x = 0; x < (OW + 3) / 4 * 4; ++x) acc[x] = bs;
#pragma unroll
            for (int kr = 0; kr < 3; ++kr) {
                const uint32_t wk = __ldg(p.wrow + c * 3 + kr);
                const int iy = S * r + kr - 1;
                uint32_t A[NA + 1];
                if (iy >= 0 && iy < p.H) {
                    const int sb = pl * P + iy * W - 1;              // byte of col -1 (may be -1: the 16 bytes in front)
                    const uint32_t* wp = reinterpret_cast<const uint32_t*>(in + (sb & ~3));
                    const uint32_t sh = 8u * (uint32_t)(sb & 3);
                    uint32_t Wd[NA + 1];
#pragma unroll
                    for (int i = 0; i <= NA; ++i) Wd[i] = wp[i];
#pragma unroll
                    for (int i = 0; i < NA; ++i) A[i] = __funnelshift_r(Wd[i], Wd[i + 1], sh);
                    // the zero point left of the first and right of the last column
                    A[0] = (A[0] & 0xffffff00u) | (p.pad_word & 0xffu);
                    constexpr int rb = W + 1;
                    A[rb / 4] = (A[rb / 4] & ~(0xffu << (8 * (rb % 4)))) | (p.pad_word & (0xffu << (8 * (rb % 4))));
                } else {
#pragma unroll
                    for (int i = 0; i < NA; ++i) A[i] = p.pad_word;
                }
                A[NA] = 0;
#pragma unroll
                for (int x = 0; x < OW; ++x) {
                    const int j = (S * x) / 4, o = (S * x) % 4;
                    const uint32_t win = o == 0 ? A[j] : __byte_perm(A[j], A[j + 1], o == 1 ? 0x4321 : (o == 2 ? 0x5432 : 0x6543));
                    acc[x] = dw_dp4a<XU8>(win, wk, acc[x]);
                }
            }
            // OW results to out + pl * PO + r * OW, which has no alignment: single bytes (pairs when every row starts on an even byte)
            uint8_t* dst = out + pl * PO + r * OW;
#pragma unroll
            for (int j = 0; j < (OW + 3) / 4; ++j) {
                const int a4[4] = {acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]};
                const uint32_t pk = dw_requant4<LEAN, false>(a4, m, cp, p);
                if (OW % 2 == 0) {
                    if (4 * j + 1 < OW) *reinterpret_cast<uint16_t*>(dst + 4 * j) = (uint16_t)(pk & 0xffffu);
                    if (4 * j + 3 < OW) *reinterpret_cast<uint16_t*>(dst + 4 * j + 2) = (uint16_t)(pk >> 16);
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (4 * j + k < OW) dst[4 * j + k] = (uint8_t)(pk >> (8 * k));
                }
            }
        }
        if (whole) ptx::fence_proxy_async_smem();
        __syncthreads();
        if (whole) {
            if (t == 0) ptx::bulk_s2g(p.y + (size_t)b * a.out_bytes, ptx::smem_u32(out), (uint32_t)a.out_bytes);
        } else {
            uint8_t* dstg = p.y + (size_t)b * a.out_bytes;
            for (int i = t; i < n_pl * PO; i += 256) dstg[i] = out[i];
        }
        ibuf = ibuf == 2 ? 0 : ibuf + 1;
        c += c_step; if (c >= p.C) c -= p.C;
    }
    if (t == 0) {
        ptx::bulk_wait_all();
        if (*abort_flag) atomicExch(a.status, (int)DEV_ERR_WAIT_TIMEOUT);
    }
}

// Stride 1 on planes whose rows are not whole words (14 x 14, 7 x 7, odd sizes), "flat" form.  The tensor is one run of
// bytes and a thread owns one aligned 4-byte word of the OUTPUT: four consecutive flat positions, which may lie in two
// rows or even two planes.  Output position f reads input bytes f - W - 1 .. f - W + 1, f - 1 .. f + 1 and
// f + W - 1 .. f + W + 1, so the three filter rows of a word are three 6-byte runs of the input at fixed distances from
// the word: two or three aligned words each (L1 serves the overlap between neighbouring threads), a funnel shift to
// the run's first byte and three byte permutes give the four 3-byte windows.  Taps that fall outside the plane
// (first / last row, first / last column) are replaced by the input zero point through per-thread byte masks.
// The pattern of rows, columns and planes within a word repeats every lcm(H*W, 4) bytes: a thread keeps its position
// within that period for the whole launch (the masks are computed once) and strides over the tensor period by period.
// Loads and stores are whole aligned words, consecutive threads touch consecutive words.
// TWO: a word may span two planes (H*W is not a multiple of 4), i.e. two channels with their own weights and constants.
template <bool XU8, bool LEAN, bool TWO>
__global__ void __launch_bounds__(256) qdwconv3x3_flat_kernel(const QDwArgs p, int Lw, int Lp, int kgroups) {
    const int t = threadIdx.x;
    if (t >= Lw * kgroups) return;
    const int P = p.H * p.W;
    const int g = t / Lw, wj = t - g * Lw;
    // per-thread geometry of the word's four bytes
    uint32_t m[3][4];
    int second = 4;                        // first byte that belongs to the word's second plane (4: none)
    int pp0 = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int fb = 4 * wj + k, pl = fb / P, f = fb - pl * P;
        const int row = f / p.W, col = f - row * p.W;
        if (k == 0) pp0 = pl;
        else if (pl != pp0 && second == 4) second = k;
        const uint32_t cm = (col > 0 ? 0x000000ffu : 0u) | 0x0000ff00u | (col < p.W - 1 ? 0x00ff0000u : 0u);
        m[0][k] = row > 0 ? cm : 0u; m[1][k] = cm; m[2][k] = row < p.H - 1 ? cm : 0u;
    }
    // the three runs start o = (r - 1) * W - 1 bytes from the word: word offset q, byte rsh within it
    int q[3]; uint32_t rsh[3];
#pragma unroll
    for (int r = 0; r < 3; ++r) {
        const int o = (r - 1) * p.W - 1;
        q[r] = o >= 0 ? o >> 2 : -((3 - o) >> 2);
        rsh[r] = (uint32_t)(o - 4 * q[r]);
    }
    const int NB = p.planes * P;                         // bytes of the tensor (the host admits less than 2^31)
    const int NW = (NB + 3) >> 2;
    const uint32_t* x32 = reinterpret_cast<const uint32_t*>(p.x);
    uint32_t* y32 = reinterpret_cast<uint32_t*>(p.y);
    const int step_planes = (int)gridDim.x * kgroups * Lp;
    const int stepC = step_planes % p.C;
    int cA = (int)(((long long)((int)blockIdx.x * kgroups + g) * Lp + pp0) % p.C);
    const uint32_t hi4 = p.act == ZANT_QACT_RELU6 ? 0x01010101u * (uint32_t)(p.six & 255) : 0x7f7f7f7fu;
    const Requant rq{p.y_scale, p.y_zp, p.act, p.lut};
    for (int J = ((int)blockIdx.x * kgroups + g) * Lw + wj; J < NW; J += (int)gridDim.x * kgroups * Lw) {
        // channel constants of the word's plane(s)
        const int cB = cA + 1 == p.C ? 0 : cA + 1;
        uint32_t wa[3], wb[3];
        float mA, mB; int bA, bB;
#pragma unroll
        for (int r = 0; r < 3; ++r) wa[r] = __ldg(p.wrow + cA * 3 + r);
        mA = __ldg(p.mult + cA); bA = __ldg(p.bias + cA);
        if (TWO) {
#pragma unroll
            for (int r = 0; r < 3; ++r) wb[r] = __ldg(p.wrow + cB * 3 + r);
            mB = __ldg(p.mult + cB); bB = __ldg(p.bias + cB);
        }
        cA += stepC; if (cA >= p.C) cA -= p.C;
        // The three runs' words.  Words whose every load lies inside the tensor (all but the first and last few of the launch)
        // take plain loads in one straight block; the others check every index.
        uint32_t wA[3], wB[3], wC[3];
        if (J + q[0] >= 0 && (long long)(J + q[2] + 3) * 4 <= (long long)NB) {
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                const uint32_t* src = x32 + (J + q[r]);
                wA[r] = __ldg(src); wB[r] = __ldg(src + 1);
                wC[r] = rsh[r] == 3u ? __ldg(src + 2) : 0u;
            }
        } else {
            auto ldw = [&](int idx) -> uint32_t {
                if (idx < 0 || idx >= NW) return p.pad_word;
                if ((long long)(idx + 1) * 4 <= (long long)NB) return __ldg(x32 + idx);
                uint32_t v = 0;
                for (int i = 0; idx * 4 + i < NB; ++i) v |= (uint32_t)__ldg(p.x + (size_t)idx * 4 + i) << (8 * i);
                return v;
            };
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                wA[r] = ldw(J + q[r]); wB[r] = ldw(J + q[r] + 1);
                wC[r] = rsh[r] == 3u ? ldw(J + q[r] + 2) : 0u;
            }
        }
        int acc[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] = (TWO && k >= second) ? bB : bA;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const uint32_t X0 = __funnelshift_r(wA[r], wB[r], 8u * rsh[r]), X1 = __funnelshift_r(wB[r], wC[r], 8u * rsh[r]);
            const uint32_t w[4] = {X0, __byte_perm(X0, X1, 0x4321), __byte_perm(X0, X1, 0x5432), __byte_perm(X0, X1, 0x6543)};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t v = (w[k] & m[r][k]) | (p.pad_word & ~m[r][k]);
                acc[k] = dw_dp4a<XU8>(v, (TWO && k >= second) ? wb[r] : wa[r], acc[k]);
            }
        }
        uint32_t pk;
        if (LEAN) {
            pk = pack_act_s8x4(rq_round(acc[0], mA), rq_round(acc[1], (TWO && 1 >= second) ? mB : mA),
                               rq_round(acc[2], (TWO && 2 >= second) ? mB : mA), rq_round(acc[3], (TWO && 3 >= second) ? mB : mA), p.act_mode != 0, hi4);
            if (p.lut) pk = lut4(p.lut, pk);
        } else {
            pk = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float mk = (TWO && k >= second) ? mB : mA;
                const int qv = p.out_u8 ? requant_one<true>(acc[k], mk, rq) : requant_one<false>(acc[k], mk, rq);
                pk |= (uint32_t)(qv & 255) << (8 * k);
            }
        }
        if ((long long)J * 4 + 4 <= (long long)NB) y32[J] = pk;
        else for (int i = 0; J * 4 + i < NB; ++i) p.y[(size_t)J * 4 + i] = (uint8_t)(pk >> (8 * i));
    }
}

// Shapes the kernel covers: 3x3, group == channels == filters, pads 1 on every side, dilation 1,
// stride 1 or 2 on both axes (even sizes for stride 2), at most 128 output columns, weight zero points 0.
inline bool qdwconv_eligible(const ConvGeom& g, bool w_zp_all_zero) {
    if (!w_zp_all_zero || g.G != g.C || g.M != g.C || g.Cg != 1 || g.KH != 3 || g.KW != 3) return false;
    if (g.dh != 1 || g.dw != 1 || g.pt != 1 || g.pl != 1 || g.pb != 1 || g.pr != 1) return false;
    if (g.sh != g.sw || (g.sh != 1 && g.sh != 2)) return false;
    if (g.OW > 128) return false;
    if (g.sh == 2 && (g.W != 2 * g.OW || g.H != 2 * g.OH)) return false;   // even sizes: no pixel right of / below the last window
    return (long long)g.N * g.C <= 0x7fffffffLL;
}

// Host constants: filter rows packed for dp4a and the bias with the input zero point folded in.
inline void qdwconv_prepare(const ConvGeom& g, const int8_t* w, const int32_t* bias, int x_zp, std::vector<uint32_t>& wrow, std::vector<int32_t>& bias_f) {
    wrow.assign((size_t)g.C * 3, 0);
    bias_f.assign(g.C, 0);
    for (int c = 0; c < g.C; ++c) {
        int sum = 0;
        for (int kh = 0; kh < 3; ++kh) {
            uint32_t word = 0;
            for (int kw = 0; kw < 3; ++kw) {
                const int8_t v = w[(size_t)c * 9 + kh * 3 + kw];
                word |= (uint32_t)(uint8_t)v << (8 * kw);
                sum += v;
            }
            wrow[(size_t)c * 3 + kh] = word;
        }
        bias_f[c] = (bias ? bias[c] : 0) - x_zp * sum;
    }
}

template <int STRIDE, bool ALIGNED>
inline int32_t qdwconv_launch_s(zant_ctx* ctx, const QDwArgs& a, int grid, bool x_u8, bool lean) {
    if (x_u8) { if (lean) qdwconv3x3_kernel<STRIDE, true, true, ALIGNED><<<grid, 256, 0, ctx->stream>>>(a); else qdwconv3x3_kernel<STRIDE, true, false, ALIGNED><<<grid, 256, 0, ctx->stream>>>(a); }
    else { if (lean) qdwconv3x3_kernel<STRIDE, false, true, ALIGNED><<<grid, 256, 0, ctx->stream>>>(a); else qdwconv3x3_kernel<STRIDE, false, false, ALIGNED><<<grid, 256, 0, ctx->stream>>>(a); }
    return check_launch(ctx, "qdwconv3x3_kernel");
}

template <int STRIDE, bool XU8, bool LEAN>
inline int32_t qdwconv_launch_smem_t(zant_ctx* ctx, const QDwArgs& a, int grid, size_t smem, bool stage_in) {
    if (stage_in) {
        ZB_SMEM_ATTR(ctx, (qdwconv3x3_kernel<STRIDE, XU8, LEAN, true, true, true>), 96 * 1024);
        qdwconv3x3_kernel<STRIDE, XU8, LEAN, true, true, true><<<grid, 256, smem, ctx->stream>>>(a);
    } else {
        ZB_SMEM_ATTR(ctx, (qdwconv3x3_kernel<STRIDE, XU8, LEAN, true, true, false>), 96 * 1024);
        qdwconv3x3_kernel<STRIDE, XU8, LEAN, true, true, false><<<grid, 256, smem, ctx->stream>>>(a);
    }
    return check_launch(ctx, "qdwconv3x3_kernel<smem>");
}

inline int32_t qdwconv_launch_smem(zant_ctx* ctx, const QDwArgs& a, int grid, size_t smem, int stride, bool x_u8, bool lean, bool stage_in) {
    if (stride == 1) {
        if (x_u8) return lean ? qdwconv_launch_smem_t<1, true, true>(ctx, a, grid, smem, stage_in) : qdwconv_launch_smem_t<1, true, false>(ctx, a, grid, smem, stage_in);
        return lean ? qdwconv_launch_smem_t<1, false, true>(ctx, a, grid, smem, stage_in) : qdwconv_launch_smem_t<1, false, false>(ctx, a, grid, smem, stage_in);
    }
    if (x_u8) return lean ? qdwconv_launch_smem_t<2, true, true>(ctx, a, grid, smem, stage_in) : qdwconv_launch_smem_t<2, true, false>(ctx, a, grid, smem, stage_in);
    return lean ? qdwconv_launch_smem_t<2, false, true>(ctx, a, grid, smem, stage_in) : qdwconv_launch_smem_t<2, false, false>(ctx, a, grid, smem, stage_in);
}

// x and y must be 4-byte aligned (the caller checks with qdwconv_ptr_ok).
inline bool qdwconv_ptr_ok(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

inline int32_t run_qdwconv(zant_ctx* ctx, const ConvGeom& g, const void* x, bool x_u8, int x_zp, const uint32_t* wrow_dev, const float* mult_dev,
                           const int32_t* bias_dev, void* y, bool y_u8, const Requant& rq, bool mult_finite, const int32_t* cap_dev = nullptr) {
    QDwArgs a{};
    a.x = (const uint8_t*)x; a.y = (uint8_t*)y; a.wrow = wrow_dev; a.mult = mult_dev; a.bias = bias_dev;
    a.planes = g.N * g.C; a.C = g.C; a.H = g.H; a.W = g.W; a.OH = g.OH; a.OW = g.OW;
    a.x_bytes = (long long)g.N * g.C * g.H * g.W;
    const int cols = (g.OW + 3) / 4;
    for (a.log2LW = 0; (1 << a.log2LW) < cols; ++a.log2LW) {}
    a.pad_word = 0x01010101u * (uint32_t)(x_zp & 255);
    a.y_scale = rq.y_scale; a.y_zp = rq.y_zp; a.act = rq.act; a.out_u8 = y_u8 ? 1 : 0; a.lut = rq.lut;
    const bool lean = !y_u8 && rq.y_zp == 0 && mult_finite;
    if (lean) a.six = lean_six(rq.y_scale);
    a.cap = cap_dev;
    a.act_mode = rq.act == ZANT_QACT_NONE ? 0 : (cap_dev ? 1 : 2);
    const int ppw = 32 >> a.log2LW;
    const long long groups = ((long long)a.planes + ppw - 1) / ppw;
    const int grid = (int)std::min<long long>((groups + 7) / 8, (long long)ctx->sm_count * 16);
    if (grid == 0) return ZANT_OK;
    if (g.sh == 1 && g.W % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 7u) == 0 && (reinterpret_cast<uintptr_t>(y) & 7u) == 0) {
        // 8 columns per lane
        const int cols8 = g.W / 8;
        for (a.log2LW = 0; (1 << a.log2LW) < cols8; ++a.log2LW) {}
        if (a.log2LW <= 5) {
            const int ppw8 = 32 >> a.log2LW;
            const long long groups8 = ((long long)a.planes + ppw8 - 1) / ppw8;
            const int grid8 = (int)std::min<long long>((groups8 + 7) / 8, (long long)ctx->sm_count * 16);
            if (x_u8) { if (lean) qdwconv3x3_s1w8_kernel<true, true><<<grid8, 256, 0, ctx->stream>>>(a); else qdwconv3x3_s1w8_kernel<true, false><<<grid8, 256, 0, ctx->stream>>>(a); }
            else { if (lean) qdwconv3x3_s1w8_kernel<false, true><<<grid8, 256, 0, ctx->stream>>>(a); else qdwconv3x3_s1w8_kernel<false, false><<<grid8, 256, 0, ctx->stream>>>(a); }
            return check_launch(ctx, "qdwconv3x3_s1w8_kernel");
        }
    }
    const bool aligned = g.W % 4 == 0 && g.OW % 4 == 0;
    const bool rows_s1 = g.sh == 1 && (g.W == 28 || g.W == 14 || g.W == 7) && g.OW == g.W && g.OH == g.H;
    const bool rows_s2 = g.sh == 2 && (g.W == 28 || g.W == 14) && g.OW == g.W / 2 && g.OH == (g.H + 1) / 2;
    if ((rows_s1 || rows_s2) && g.OH <= 64 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0) {
        // small planes: batches of whole planes through shared memory, a thread per output row
        const int P = g.H * g.W, PO = g.OH * g.OW;
        int unit = 16;                                       // planes per batch come in units that make both batch sizes multiples of 16 bytes
        while (unit > 1 && (P * (unit / 2)) % 16 == 0 && (PO * (unit / 2)) % 16 == 0) unit /= 2;
        QDwRowsArgs ra{};
        ra.p = a;
        ra.PB = 256 / g.OH / unit * unit;
        if (ra.PB >= unit && a.planes >= 4 * ra.PB) {
            ra.batches = (a.planes + ra.PB - 1) / ra.PB;
            ra.buf_bytes = ra.PB * P;
            ra.out_bytes = ra.PB * PO;
            ra.status = ctx->status_word;
            const int in_stride = (ra.buf_bytes + 32 + 127) / 128 * 128, out_stride = (ra.out_bytes + 127) / 128 * 128;
            const size_t smem = (size_t)3 * in_stride + 2 * out_stride + 32;
            const int rgrid = (int)std::min<long long>(ra.batches, (long long)ctx->sm_count * 8);
            auto go = [&](auto kernel) -> int32_t {
                kernel<<<rgrid, 256, smem, ctx->stream>>>(ra);
                return check_launch(ctx, "qdwconv3x3_rows_kernel");
            };
            auto pick = [&](auto w_tag, auto s_tag) -> int32_t {
                constexpr int KW = decltype(w_tag)::value, KS = decltype(s_tag)::value;
                if (x_u8) return lean ? go(qdwconv3x3_rows_kernel<true, true, KW, KS>) : go(qdwconv3x3_rows_kernel<true, false, KW, KS>);
                return lean ? go(qdwconv3x3_rows_kernel<false, true, KW, KS>) : go(qdwconv3x3_rows_kernel<false, false, KW, KS>);
            };
            if (smem <= 48 * 1024) {
                using std::integral_constant;
                if (rows_s1 && g.W == 28) return pick(integral_constant<int, 28>{}, integral_constant<int, 1>{});
                if (rows_s1) return g.W == 14 ? pick(integral_constant<int, 14>{}, integral_constant<int, 1>{}) : pick(integral_constant<int, 7>{}, integral_constant<int, 1>{});
                return g.W == 28 ? pick(integral_constant<int, 28>{}, integral_constant<int, 2>{}) : pick(integral_constant<int, 14>{}, integral_constant<int, 2>{});
            }
        }
    }
    if (!aligned && g.sh == 1) {
        // rows that are not whole words, stride 1: the flat form, when its period fits a CTA
        const long long P = (long long)g.H * g.W, nb = (long long)a.planes * P;
        const int Lp = P % 4 == 0 ? 1 : (P % 2 == 0 ? 2 : 4);
        const long long Lw = P * Lp / 4;
        if (P >= 8 && Lw <= 256 && nb < 0x7fffffffLL - 64) {      // P >= 8: a word spans at most two planes
            const int kg = (int)std::max<long long>(1, 256 / Lw);
            const long long periods = ((nb + 3) / 4 + Lw - 1) / Lw;
            const int fgrid = (int)std::min<long long>((periods + kg - 1) / kg, (long long)ctx->sm_count * 8);
            auto go = [&](auto kernel) -> int32_t {
                kernel<<<fgrid, 256, 0, ctx->stream>>>(a, (int)Lw, Lp, kg);
                return check_launch(ctx, "qdwconv3x3_flat_kernel");
            };
            if (Lp == 1) {
                if (x_u8) return lean ? go(qdwconv3x3_flat_kernel<true, true, false>) : go(qdwconv3x3_flat_kernel<true, false, false>);
                return lean ? go(qdwconv3x3_flat_kernel<false, true, false>) : go(qdwconv3x3_flat_kernel<false, false, false>);
            }
            if (x_u8) return lean ? go(qdwconv3x3_flat_kernel<true, true, true>) : go(qdwconv3x3_flat_kernel<true, false, true>);
            return lean ? go(qdwconv3x3_flat_kernel<false, true, true>) : go(qdwconv3x3_flat_kernel<false, false, true>);
        }
    }
    if (!aligned) {
        // rows that are not whole words: stage the planes through shared memory when a pass (8 warps x planes per warp) fits
        const bool stage_in = g.W % 4 != 0;      // input rows of whole words are read straight from global memory
        const int Wp = (g.W + 7) / 8 * 8, OWp = (g.OW + 3) / 4 * 4;
        const size_t smem = (size_t)8 * ppw * ((stage_in ? (size_t)g.H * Wp : 0) + (size_t)g.OH * OWp);
        if (smem <= 96 * 1024) {
            const int sgrid = (int)std::min<long long>((groups + 7) / 8, (long long)ctx->sm_count * (stage_in ? 4 : 8));
            return qdwconv_launch_smem(ctx, a, sgrid, smem, g.sh, x_u8, lean, stage_in);
        }
    }
    if (g.sh == 1) return aligned ? qdwconv_launch_s<1, true>(ctx, a, grid, x_u8, lean) : qdwconv_launch_s<1, false>(ctx, a, grid, x_u8, lean);
    return aligned ? qdwconv_launch_s<2, true>(ctx, a, grid, x_u8, lean) : qdwconv_launch_s<2, false>(ctx, a, grid, x_u8, lean);
}

}  // namespace zb
