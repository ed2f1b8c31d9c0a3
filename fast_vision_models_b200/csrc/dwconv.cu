// Depthwise RxS convolution, NHWC fp16, weights [R,S,C], fused bias + activation and an optional fused squeeze
// (per-(image, channel) sums of the rounded outputs, the first half of a squeeze-excite block).
//
// Both kernels work on a tile of output pixels x a block of channels whose input patch (with its filter border) is
// brought into shared memory by ONE bulk tensor copy (TMA, 4-D map over the NHWC activation): padding is the copy's
// zero fill, the SM spends no instruction on addresses or bounds of the input, and every input byte crosses L2 -> SM
// about once. Several small CTAs share an SM, so one CTA's copy is in flight while others compute.
//
//   dw_tile_kernel<S, SW, ACT>   square 3/5/7-tap filters, stride 1 or 2, no dilation (every depthwise layer of
//                                EfficientNet and ConvNeXt). Thread = 8 channels x 8 consecutive output columns of one
//                                output row; one kernel row of weights and the 64 accumulators live in registers.
//                                Arithmetic of the reference's dwconv2 (classification/fast/csrc/r3.cu:354-415, its
//                                default mode): fp16x2 FMAs within a kernel row starting from zero, fp32 across rows,
//                                result rounded to fp16, then the activation.
//   dw_any_kernel                any filter size, stride and dilation (the contract of segx::dwconv, segmentation/fast/
//                                seg_kernels.cu:124-158, and of clf::dwconv, classification/fast/csrc/fused_conv.cu:
//                                428-475): thread = 8 channels x one output pixel, taps looped at run time, fp32
//                                accumulation throughout: acc = bias; acc += x * w per tap; y = half(act(acc)).
//
// Channel blocks are 64, 32, 16 or 8 channels wide, whichever wastes the fewest lanes for the layer's channel count
// (C = 96 takes three blocks of 32; out-of-range channels of the last block arrive as zeros and are not stored).
// Fused squeeze: every CTA reduces its outputs per channel in a fixed order and writes one fp32 partial sum per channel
// to its own slot of `pool_partial` [N][slots][C]; the squeeze-excite gate adds the slots in order. No atomics: the
// result does not depend on scheduling.
#include <cuda.h>

#include <cstdint>
#include <cstring>

#include "fvm_internal.h"
#include "ptx_sm100.cuh"

namespace fvm {

static constexpr int DW_THREADS = 128;
// Output columns per thread in the tile kernel, per filter size, as measured on B200 (N = 64; 3x3 C=192 95x95:
// 119 us with 4 columns against 131 with 8; 5x5 C=336 48x48: 82 against 137 the other way round; 7x7 C=96 56x56: 64
// against 76): narrow strips keep more CTAs on an SM, wide ones re-use each staged input vector for more outputs.
static constexpr int dw_tw(int S) { return S == 5 ? 8 : 4; }
static constexpr int DW_SMEM_LIMIT = 96 * 1024; // per CTA: at least two CTAs per SM
static constexpr int STATUS_WAIT_DW = 0x105;

struct DwParams {
    int H, W, C, R, S, P, Q;
    int sh, sw, ph, pw, dh, dw;
    int cbv;                 // channel vectors (8 channels each) per block: 8, 4, 2 or 1
    int px, py;              // thread grid over the tile: px x py "cells" per channel vector (px * py * cbv = 128)
    int tiles_x, tiles_y, vblocks;
    int tile_h, tile_w;      // staged input patch in pixels
    int act;
    long long ldy;
    int* status;
};

__device__ __forceinline__ void dw_decode_block(const DwParams& p, int& tx, int& ty, int& vb) {
    int bid = blockIdx.x;
    tx = bid % p.tiles_x;
    bid /= p.tiles_x;
    ty = bid % p.tiles_y;
    vb = bid / p.tiles_y;
}

// Brings the input patch of this CTA's tile into shared memory: (channels vb*cbv*8 .., columns w0 .., rows h0 .., image
// n); coordinates outside the tensor are filled with zeros by the copy. dw_stage_issue starts the copy (one thread),
// dw_stage_wait joins the CTA and waits for it; returns false if the bounded wait ran out.
__device__ __forceinline__ void dw_stage_issue(const CUtensorMap* tmap, const DwParams& p, uint32_t smem0, uint32_t bar,
                                               int vb, int w0, int h0, int n, volatile int* abort_flag) {
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar, 1);
        mbar_fence_init();
        mbar_expect_tx(bar, static_cast<uint32_t>(p.tile_h * p.tile_w * p.cbv) * 16u);
        tma_load_4d(smem0, tmap, bar, vb * p.cbv * 8, w0, h0, n);
    }
}
__device__ __forceinline__ bool dw_stage_wait(const DwParams& p, uint32_t bar, volatile int* abort_flag) {
    __syncthreads();
    if (!mbar_wait<32>(bar, 0u, abort_flag)) {
        if (threadIdx.x == 0) atomicExch(p.status, STATUS_WAIT_DW);
        return false;
    }
    return true;
}

// Per-channel sums of this CTA's outputs, reduced over the cells in a fixed order, into this CTA's slot.
__device__ __forceinline__ void dw_pool_write(const DwParams& p, float* pool_s, const float (&psum)[8], bool active, int cell,
                                              int vv, int vb, long long n, int slot, float* __restrict__ pool_partial) {
    const int cb = p.cbv * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) pool_s[cell * cb + vv * 8 + k] = active ? psum[k] : 0.f;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < cb) {
        const int cells = DW_THREADS / p.cbv;
        float s = 0.f;
        for (int i = 0; i < cells; ++i) s += pool_s[i * cb + threadIdx.x];
        const int c = vb * cb + threadIdx.x;
        if (c < p.C) pool_partial[(n * (p.tiles_x * p.tiles_y) + slot) * p.C + c] = s;
    }
}

// ACT: activation known at compile time (0 none, 1 relu, 3 silu) or -1 = use the run-time code.
template <int S, int SW, int ACT, int TW>
__global__ void __launch_bounds__(DW_THREADS)
dw_tile_kernel(const __grid_constant__ CUtensorMap tmap_x, const __half* __restrict__ w, const __half* __restrict__ bias,
               __half* __restrict__ y, float* __restrict__ pool_partial, const DwParams p) {
    extern __shared__ __align__(128) uint8_t dw_smem[];
    const uint32_t smem0 = (smem_u32(dw_smem) + 127u) & ~127u;
    const uint32_t tile_bytes = static_cast<uint32_t>(p.tile_h * p.tile_w * p.cbv) * 16u;
    const uint32_t bar = smem0 + tile_bytes;
    uint8_t* after = dw_smem + (smem0 - smem_u32(dw_smem)) + tile_bytes;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(after + 8);
    float* pool_s = reinterpret_cast<float*>(after + 16);

    int tx, ty, vb;
    dw_decode_block(p, tx, ty, vb);
    const long long n = blockIdx.y;
    const int TWB = p.px * TW, TH = p.py;
    const int p0 = ty * TH, q0 = tx * TWB;
    dw_stage_issue(&tmap_x, p, smem0, bar, vb, q0 * SW - p.pw, p0 * p.sh - p.ph, static_cast<int>(n), abort_flag);
    // the block's S x S x (cbv * 8) weights: [tap][channel vector], copied while the input patch is in flight
    const uint32_t w_s = smem_u32(pool_s) + DW_THREADS * 8 * 4;
    {
        uint4* w_dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pool_s) + DW_THREADS * 8 * 4);
        const int cvb = p.C >> 3;
        for (int i = threadIdx.x; i < S * S * p.cbv; i += DW_THREADS) {
            const int tap = i / p.cbv, wv = vb * p.cbv + i % p.cbv;
            w_dst[i] = wv < cvb ? __ldg(reinterpret_cast<const uint4*>(w + static_cast<long long>(tap) * p.C + wv * 8))
                                : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    if (!dw_stage_wait(p, bar, abort_flag)) return;

    const int vv = threadIdx.x % p.cbv;
    const int cell = threadIdx.x / p.cbv;
    const int sx = cell % p.px, sy = cell / p.px;
    const int v = vb * p.cbv + vv;
    const int pr = p0 + sy, qs = q0 + sx * TW;
    const bool active = v < (p.C >> 3) && pr < p.P && qs < p.Q;
    float psum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) {
        float acc[TW][8];                   // fp32 accumulators
        {
            float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (bias) {
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + v * 8));
                f32_add_h2(b8[0], b8[1], bv.x); f32_add_h2(b8[2], b8[3], bv.y);
                f32_add_h2(b8[4], b8[5], bv.z); f32_add_h2(b8[6], b8[7], bv.w);
            }
#pragma unroll
            for (int j = 0; j < TW; ++j)
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[j][k] = b8[k];
        }
        constexpr int L = (TW - 1) * SW + S;      // staged columns one kernel row of this thread's strip reads
        const uint32_t pix = static_cast<uint32_t>(p.cbv) * 16u;
#pragma unroll(S == 3 ? 3 : 1)
        for (int r = 0; r < S; ++r) {          // square filter: R == S; short filters unrolled (next row's loads issue early)
            uint4 wr[S];                       // this kernel row of the block's weights, from shared memory
#pragma unroll
            for (int s2 = 0; s2 < S; ++s2) wr[s2] = lds128(w_s + static_cast<uint32_t>((r * S + s2) * p.cbv + vv) * 16u);
            __half2 racc[TW][4];
#pragma unroll
            for (int j = 0; j < TW; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k) racc[j][k] = __float2half2_rn(0.f);
            const uint32_t row_addr = smem0 + static_cast<uint32_t>((sy * p.sh + r) * p.tile_w + sx * TW * SW) * pix +
                                      static_cast<uint32_t>(vv) * 16u;
#pragma unroll
            for (int l = 0; l < L; ++l) {
                const uint4 xv = lds128(row_addr + static_cast<uint32_t>(l) * pix);
                const __half2* hx = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                for (int j = 0; j < TW; ++j) {
                    const int s2 = l - j * SW;          // compile-time after unrolling
                    if (s2 >= 0 && s2 < S) {
                        const __half2* hw = reinterpret_cast<const __half2*>(&wr[s2]);
#pragma unroll
                        for (int k = 0; k < 4; ++k) racc[j][k] = __hfma2(hx[k], hw[k], racc[j][k]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < TW; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    f32_add_h2(acc[j][2 * k], acc[j][2 * k + 1], *reinterpret_cast<const uint32_t*>(&racc[j][k]));
        }
#pragma unroll
        for (int j = 0; j < TW; ++j) {
            const int q = qs + j;
            if (q < p.Q) {
                __align__(16) __half2 o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    // the sum is rounded to fp16 first; relu acts on the fp16 pair, other activations are evaluated
                    // in fp32 on the rounded value and rounded again (reference: r3.cu:404-413)
                    o[k] = __floats2half2_rn(acc[j][2 * k], acc[j][2 * k + 1]);
                    if (ACT == 1) {
                        o[k] = __hmax2(o[k], __float2half2_rn(0.f));
                    } else if (ACT == 3) {      // SiLU on the pair in fp32: packed multiplies, ex2 / rcp per element
                        const uint32_t sv = f2_to_h2(f2_silu(h2_to_f2(*reinterpret_cast<const uint32_t*>(&o[k]))));
                        o[k] = *reinterpret_cast<const __half2*>(&sv);
                    } else if (ACT != 0) {
                        const float2 f = __half22float2(o[k]);
                        o[k] = __floats2half2_rn(act_f(f.x, p.act), act_f(f.y, p.act));
                    }
                    if (pool_partial) {
                        const float2 f = __half22float2(o[k]);
                        psum[2 * k] += f.x;
                        psum[2 * k + 1] += f.y;
                    }
                }
                *reinterpret_cast<uint4*>(y + ((n * p.P + pr) * p.Q + q) * p.ldy + v * 8) = *reinterpret_cast<uint4*>(o);
            }
        }
    }
    if (pool_partial) dw_pool_write(p, pool_s, psum, active, cell, vv, vb, n, ty * p.tiles_x + tx, pool_partial);
}

// Any filter, stride and dilation: thread = 8 channels x one output pixel of the tile; fp32 accumulation.
__global__ void __launch_bounds__(DW_THREADS)
dw_any_kernel(const __grid_constant__ CUtensorMap tmap_x, const __half* __restrict__ w, const __half* __restrict__ bias,
              __half* __restrict__ y, float* __restrict__ pool_partial, const DwParams p) {
    extern __shared__ __align__(128) uint8_t dw_smem[];
    const uint32_t smem0 = (smem_u32(dw_smem) + 127u) & ~127u;
    const uint32_t tile_bytes = static_cast<uint32_t>(p.tile_h * p.tile_w * p.cbv) * 16u;
    const uint32_t bar = smem0 + tile_bytes;
    uint8_t* after = dw_smem + (smem0 - smem_u32(dw_smem)) + tile_bytes;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(after + 8);
    float* pool_s = reinterpret_cast<float*>(after + 16);

    int tx, ty, vb;
    dw_decode_block(p, tx, ty, vb);
    const long long n = blockIdx.y;
    const int p0 = ty * p.py, q0 = tx * p.px;
    dw_stage_issue(&tmap_x, p, smem0, bar, vb, q0 * p.sw - p.pw, p0 * p.sh - p.ph, static_cast<int>(n), abort_flag);
    if (!dw_stage_wait(p, bar, abort_flag)) return;

    const int vv = threadIdx.x % p.cbv;
    const int cell = threadIdx.x / p.cbv;
    const int cx = cell % p.px, cy = cell / p.px;
    const int v = vb * p.cbv + vv;
    const int pr = p0 + cy, q = q0 + cx;
    const bool active = v < (p.C >> 3) && pr < p.P && q < p.Q;
    float psum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (bias) {
            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + v * 8));
            const __half2* hb = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(hb[k]);
                acc[2 * k] = f.x;
                acc[2 * k + 1] = f.y;
            }
        }
        const uint32_t pix = static_cast<uint32_t>(p.cbv) * 16u;
        for (int r = 0; r < p.R; ++r) {
            const uint32_t row_addr = smem0 + static_cast<uint32_t>((cy * p.sh + r * p.dh) * p.tile_w + cx * p.sw) * pix +
                                      static_cast<uint32_t>(vv) * 16u;
            const __half* wrow = w + static_cast<long long>(r) * p.S * p.C + v * 8;
            for (int s2 = 0; s2 < p.S; ++s2) {
                const uint4 xv = lds128(row_addr + static_cast<uint32_t>(s2 * p.dw) * pix);
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + static_cast<long long>(s2) * p.C));
                const __half2* hx = reinterpret_cast<const __half2*>(&xv);
                const __half2* hw = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 a = __half22float2(hx[k]), b = __half22float2(hw[k]);
                    acc[2 * k] = fmaf(a.x, b.x, acc[2 * k]);
                    acc[2 * k + 1] = fmaf(a.y, b.y, acc[2 * k + 1]);
                }
            }
        }
        __align__(16) __half2 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            o[k] = __floats2half2_rn(act_f(acc[2 * k], p.act), act_f(acc[2 * k + 1], p.act));
            if (pool_partial) {
                const float2 f = __half22float2(o[k]);
                psum[2 * k] = f.x;
                psum[2 * k + 1] = f.y;
            }
        }
        *reinterpret_cast<uint4*>(y + ((n * p.P + pr) * p.Q + q) * p.ldy + v * 8) = *reinterpret_cast<uint4*>(o);
    }
    if (pool_partial) dw_pool_write(p, pool_s, psum, active, cell, vv, vb, n, ty * p.tiles_x + tx, pool_partial);
}

// Channel vectors per block: the widest block that wastes at most an eighth of its lanes on channels past C.
static int pick_cbv(int cv) {
    const int cands[4] = {8, 4, 2, 1};
    for (int i = 0; i < 4; ++i) {
        const int c = cands[i];
        const int padded = (cv + c - 1) / c * c;
        if (padded * 8 <= cv * 9) return c;
    }
    return 1;
}

struct DwPlan {
    DwParams p;
    bool tile_kernel;
    size_t smem;
};

// Tile geometry for one layer: which kernel, the channel block, the cell grid and the staged patch.
static bool dw_plan(int N, int H, int W, int C, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw, long long ldy,
                    int act, DwPlan* out) {
    DwParams& p = out->p;
    memset(&p, 0, sizeof(p));
    p.H = H; p.W = W; p.C = C; p.R = R; p.S = S;
    p.P = (H + 2 * ph - dh * (R - 1) - 1) / sh + 1;
    p.Q = (W + 2 * pw - dw * (S - 1) - 1) / sw + 1;
    if (p.P <= 0 || p.Q <= 0) return false;
    p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
    p.act = act;
    p.ldy = ldy;
    const int cv = C >> 3;
    out->tile_kernel = R == S && (S == 3 || S == 5 || S == 7) && dh == 1 && dw == 1 && sh == sw && (sw == 1 || sw == 2);
    // Candidates: channel blocks from the widest acceptable one down, cell grids px x py with px a power of two. Among
    // the candidates whose product of (useful lanes) x (useful cells: tiles overhang the map) is within 15 % of the best,
    // the one with the least staged bytes per output pixel (least border) is taken. Measured on B200: small CTAs win
    // over taller tiles with several output rows per thread (more CTAs per SM overlap one CTA's copy with the others'
    // arithmetic), so a thread keeps to one output row.
    const int unit = out->tile_kernel ? dw_tw(S) : 1;
    struct Cand { int cbv, px, py, tile_w, tile_h, tiles_x, tiles_y, vblocks; double score, cost; size_t bytes; };
    Cand cands[40];
    int nc = 0;
    double best_score = 0.0;
    for (int cbv = pick_cbv(cv); cbv >= 1 && nc < 32; cbv >>= 1) {
        const int cells = DW_THREADS / cbv;
        const int vblocks = (cv + cbv - 1) / cbv;
        const double lane_eff = static_cast<double>(cv) / (vblocks * cbv);
        for (int px = 1; px <= cells && nc < 40; px <<= 1) {
            const int py = cells / px;
            const int tile_w = (px * unit - 1) * sw + (S - 1) * dw + 1;
            const int tile_h = (py - 1) * sh + (R - 1) * dh + 1;
            const size_t bytes = static_cast<size_t>(tile_h) * tile_w * cbv * 16;
            if (tile_w > 256 || tile_h > 256 || bytes + 128 + 16 + 4096 + 6272 > static_cast<size_t>(DW_SMEM_LIMIT)) continue;
            const int tiles_x = (p.Q + px * unit - 1) / (px * unit), tiles_y = (p.P + py - 1) / py;
            const double tile_eff = static_cast<double>(p.P) * p.Q / (static_cast<double>(tiles_y) * py * tiles_x * px * unit);
            Cand c = {cbv, px, py, tile_w, tile_h, tiles_x, tiles_y, vblocks, lane_eff * tile_eff,
                      static_cast<double>(tile_h) * tile_w / (py * px * unit), bytes};
            cands[nc++] = c;
            if (c.score > best_score) best_score = c.score;
        }
        if (best_score > 0.97) break;       // narrower channel blocks only when the wide ones waste lanes
    }
    int pick = -1;
    for (int i = 0; i < nc; ++i)
        if (cands[i].score >= 0.85 * best_score && (pick < 0 || cands[i].cost < cands[pick].cost)) pick = i;
    if (pick < 0) return false;
    const Cand& c = cands[pick];
    p.cbv = c.cbv; p.px = c.px; p.py = c.py; p.tile_w = c.tile_w; p.tile_h = c.tile_h;
    p.tiles_x = c.tiles_x; p.tiles_y = c.tiles_y; p.vblocks = c.vblocks;
    out->smem = 128 + c.bytes + 16 + static_cast<size_t>(DW_THREADS) * 8 * sizeof(float) + 6272;    // + up to 49 taps x 8 vectors of weights
    (void)N;
    return true;
}

}  // namespace fvm

using namespace fvm;

extern "C" int fvm_dwconv_pool_slots(int N, int H, int W, int C, int R, int S, int ph, int pw, int sh, int sw, int dh,
                                     int dw) {
    DwPlan plan;
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || (C & 7) || R <= 0 || S <= 0 || sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || ph < 0 || pw < 0)
        return -1;
    if (!dw_plan(N, H, W, C, R, S, ph, pw, sh, sw, dh, dw, C, 0, &plan)) return -1;
    return plan.p.tiles_x * plan.p.tiles_y;
}

extern "C" int fvm_dwconv_f16(const void* x, const void* w_rsc, const void* bias, void* y, float* pool_partial, int N,
                              int H, int W, int C, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                              long long ldx, long long ldy, int act, void* stream) {
    if (!x || !w_rsc || !y || N <= 0 || N > 65535 || H <= 0 || W <= 0 || C <= 0 || (C & 7) || R <= 0 || S <= 0 ||
        sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || ph < 0 || pw < 0 || (ldx & 7) || (ldy & 7) || ldx < C || ldy < C ||
        act < 0 || act > 6)
        return FVM_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w_rsc) & 15) ||
        (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(bias) & 15) ||
        (reinterpret_cast<uintptr_t>(pool_partial) & 3))
        return FVM_ERR_ARG;
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    DwPlan plan;
    if (!dw_plan(N, H, W, C, R, S, ph, pw, sh, sw, dh, dw, ldy, act, &plan)) return FVM_ERR_ARG;
    DwParams& p = plan.p;
    p.status = st->status_dev;

    // NHWC activation as (C, W, H, N); one box = the staged patch of one tile x one channel block, zero outside
    CUtensorMap tmap;
    {
        const unsigned long long dims[4] = {static_cast<unsigned long long>(C), static_cast<unsigned long long>(W),
                                            static_cast<unsigned long long>(H), static_cast<unsigned long long>(N)};
        const unsigned long long strides[3] = {static_cast<unsigned long long>(ldx) * 2,
                                               static_cast<unsigned long long>(W) * ldx * 2,
                                               static_cast<unsigned long long>(H) * W * ldx * 2};
        const unsigned box[4] = {static_cast<unsigned>(p.cbv * 8), static_cast<unsigned>(p.tile_w),
                                 static_cast<unsigned>(p.tile_h), 1u};
        const int rc = encode_tiled_f16(&tmap, x, 4, dims, strides, box, /*swizzle128=*/false);
        if (rc != FVM_OK) return rc;
    }
    const long long bx = static_cast<long long>(p.tiles_x) * p.tiles_y * p.vblocks;
    if (bx > 0x7fffffffll) return FVM_ERR_ARG;
    const dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(N));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __half* wp = static_cast<const __half*>(w_rsc);
    const __half* bp = static_cast<const __half*>(bias);
    __half* yp = static_cast<__half*>(y);
#define DW_LAUNCH(KERNEL)                                                                                             \
    do {                                                                                                              \
        if (plan.smem > 48 * 1024 &&                                                                                  \
            cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, DW_SMEM_LIMIT) != cudaSuccess)  \
            return FVM_ERR_SETUP;                                                                                     \
        KERNEL<<<grid, DW_THREADS, plan.smem, s>>>(tmap, wp, bp, yp, pool_partial, p);                                \
    } while (0)
#define DW_ACT_TW(SV, SWV, TWV)                                               \
    do {                                                                      \
        if (act == 0) DW_LAUNCH((dw_tile_kernel<SV, SWV, 0, TWV>));           \
        else if (act == 1) DW_LAUNCH((dw_tile_kernel<SV, SWV, 1, TWV>));      \
        else if (act == 3) DW_LAUNCH((dw_tile_kernel<SV, SWV, 3, TWV>));      \
        else DW_LAUNCH((dw_tile_kernel<SV, SWV, -1, TWV>));                   \
    } while (0)
#define DW_ACT(SV, SWV) DW_ACT_TW(SV, SWV, dw_tw(SV))
    if (plan.tile_kernel) {
        if (S == 3) { if (sw == 1) DW_ACT(3, 1); else DW_ACT(3, 2); }
        else if (S == 5) { if (sw == 1) DW_ACT(5, 1); else DW_ACT(5, 2); }
        else { if (sw == 1) DW_ACT(7, 1); else DW_ACT(7, 2); }
    } else {
        DW_LAUNCH(dw_any_kernel);
    }
#undef DW_ACT
#undef DW_ACT_TW
#undef DW_LAUNCH
    count_launch();
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}
