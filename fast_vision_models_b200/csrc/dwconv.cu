// Depthwise RxS convolution, NHWC fp16, weights [R,S,C], fp32 accumulation, fused bias + activation and an optional
// fused per-(image, channel) sum of the rounded outputs (the squeeze of a squeeze-excite block).
//
// Arithmetic contract (reference: classification/fast/csrc/fused_conv.cu:428-475, dwconv_tw): acc = float(bias);
// for every in-image tap acc += float(x) * float(w); y = half(act(acc)). The reference's dwconv2 (r3.cu:335-418)
// accumulates each kernel row in fp16; this kernel keeps fp32 throughout.
//
// One thread owns 8 channels (one 16-byte vector) and TW consecutive output columns of one output row, so every input
// vector of a kernel row is loaded once and reused by up to ceil(S / stride) outputs from registers; neighbouring rows
// and strips share their halo through L1/L2. Threads of a block are consecutive in (strip, channel-vector) order with
// the channel vector fastest: every warp access is a run of contiguous 16-byte vectors.
#include <cstdint>

#include "fvm_internal.h"
#include "ptx_sm100.cuh"

namespace fvm {

static constexpr int DW_THREADS = 128;
static constexpr int DW_MAX_POOL_C = 4096;   // channels whose pool sums fit the block's shared accumulator

template <int TW>
__global__ void __launch_bounds__(DW_THREADS)
dwconv_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const __half* __restrict__ bias,
              __half* __restrict__ y, float* __restrict__ pool_sums, int H, int W, int C, int R, int S, int P, int Q,
              int sh, int sw, int ph, int pw, int dh, int dw, long long ldx, long long ldy, int act,
              long long items_per_image) {
    extern __shared__ float pool_acc[];   // [C] when pool_sums != nullptr
    const int cv = C >> 3;
    const long long n = blockIdx.y;
    if (pool_sums) {
        for (int c = threadIdx.x; c < C; c += DW_THREADS) pool_acc[c] = 0.f;
        __syncthreads();
    }
    const long long i = static_cast<long long>(blockIdx.x) * DW_THREADS + threadIdx.x;
    if (i < items_per_image) {
        const int QT = (Q + TW - 1) / TW;
        const int v = static_cast<int>(i % cv);
        long long t = i / cv;
        const int qt = static_cast<int>(t % QT);
        const int p = static_cast<int>(t / QT);
        const int q0 = qt * TW;

        float acc[TW][8];
        {
            float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (bias) {
                uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + v * 8));
                const __half2* hb = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 f = __half22float2(hb[k]);
                    b[2 * k] = f.x;
                    b[2 * k + 1] = f.y;
                }
            }
#pragma unroll
            for (int j = 0; j < TW; ++j)
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[j][k] = b[k];
        }

        const __half* ximg = x + n * H * W * ldx + v * 8;
        for (int r = 0; r < R; ++r) {
            const int h = p * sh - ph + r * dh;
            if (h < 0 || h >= H) continue;
            const __half* xrow = ximg + static_cast<long long>(h) * W * ldx;
            const __half* wrow = w + static_cast<long long>(r) * S * C + v * 8;
            if (dw == 1) {
                // sliding window: input column l of the strip feeds output j with tap s = l - j*sw
                const int L = (TW - 1) * sw + S;
                const int iw0 = q0 * sw - pw;
                for (int l = 0; l < L; ++l) {
                    const int ww = iw0 + l;
                    if (ww < 0 || ww >= W) continue;
                    const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xrow + static_cast<long long>(ww) * ldx));
                    const __half2* hx = reinterpret_cast<const __half2*>(&xv);
                    float xf[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float2 f = __half22float2(hx[k]);
                        xf[2 * k] = f.x;
                        xf[2 * k + 1] = f.y;
                    }
#pragma unroll
                    for (int j = 0; j < TW; ++j) {
                        const int s = l - j * sw;
                        if (s < 0 || s >= S) continue;
                        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + static_cast<long long>(s) * C));
                        const __half2* hw = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float2 f = __half22float2(hw[k]);
                            acc[j][2 * k] = fmaf(xf[2 * k], f.x, acc[j][2 * k]);
                            acc[j][2 * k + 1] = fmaf(xf[2 * k + 1], f.y, acc[j][2 * k + 1]);
                        }
                    }
                }
            } else {
                for (int s = 0; s < S; ++s) {
                    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + static_cast<long long>(s) * C));
                    const __half2* hw = reinterpret_cast<const __half2*>(&wv);
                    float wf[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float2 f = __half22float2(hw[k]);
                        wf[2 * k] = f.x;
                        wf[2 * k + 1] = f.y;
                    }
#pragma unroll
                    for (int j = 0; j < TW; ++j) {
                        const int ww = (q0 + j) * sw - pw + s * dw;
                        if (ww < 0 || ww >= W || q0 + j >= Q) continue;
                        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xrow + static_cast<long long>(ww) * ldx));
                        const __half2* hx = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float2 f = __half22float2(hx[k]);
                            acc[j][2 * k] = fmaf(f.x, wf[2 * k], acc[j][2 * k]);
                            acc[j][2 * k + 1] = fmaf(f.y, wf[2 * k + 1], acc[j][2 * k + 1]);
                        }
                    }
                }
            }
        }

        float psum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < TW; ++j) {
            const int q = q0 + j;
            if (q >= Q) break;
            __align__(16) __half2 o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                o[k] = __floats2half2_rn(act_f(acc[j][2 * k], act), act_f(acc[j][2 * k + 1], act));
                if (pool_sums) {
                    float2 f = __half22float2(o[k]);
                    psum[2 * k] += f.x;
                    psum[2 * k + 1] += f.y;
                }
            }
            *reinterpret_cast<uint4*>(y + ((n * P + p) * Q + q) * ldy + v * 8) = *reinterpret_cast<uint4*>(o);
        }
        if (pool_sums) {
#pragma unroll
            for (int k = 0; k < 8; ++k) atomicAdd(&pool_acc[v * 8 + k], psum[k]);
        }
    }
    if (pool_sums) {
        __syncthreads();
        for (int c = threadIdx.x; c < C; c += DW_THREADS) {
            const float s = pool_acc[c];
            if (s != 0.f) atomicAdd(pool_sums + n * C + c, s);
        }
    }
}


template <int S, int SW, int ACT>
static int launch_dw_tile_act(const __half* xp, const __half* wp, const __half* bp, __half* yp, float* pool_sums, int N,
                              int H, int W, int C, int R, int P, int Q, int sh, int ph, int pw, long long ldx,
                              long long ldy, int act, cudaStream_t st);
template <int S, int SW>
static int launch_dw_tile(const __half* xp, const __half* wp, const __half* bp, __half* yp, float* pool_sums, int N, int H,
                          int W, int C, int R, int P, int Q, int sh, int ph, int pw, long long ldx, long long ldy, int act,
                          cudaStream_t st) {
    switch (act) {
        case 0: return launch_dw_tile_act<S, SW, 0>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st);
        case 1: return launch_dw_tile_act<S, SW, 1>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st);
        case 3: return launch_dw_tile_act<S, SW, 3>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st);
        default: return launch_dw_tile_act<S, SW, -1>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st);
    }
}

// Fast path for square 3/5/7-tap kernels without dilation: S, the stride and the strip width are compile-time, so the
// accumulators (TW x 8 fp32) and one kernel row of weights (S x 8 fp32) stay in registers; every input vector of a
// kernel row is loaded and converted once and feeds up to ceil(S / stride) outputs. Loads are the only memory
// instructions in the inner loop: (TW-1)*stride + S input vectors and S weight vectors per kernel row per TW outputs.
template <int S, int SW, int TW>
__global__ void __launch_bounds__(DW_THREADS)
dwconv_fast_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const __half* __restrict__ bias,
                   __half* __restrict__ y, float* __restrict__ pool_sums, int H, int W, int C, int R, int P, int Q,
                   int sh, int ph, int pw, long long ldx, long long ldy, int act, long long items_per_image) {
    extern __shared__ float pool_acc[];   // [C] when pool_sums != nullptr
    const int cv = C >> 3;
    const long long n = blockIdx.y;
    if (pool_sums) {
        for (int c = threadIdx.x; c < C; c += DW_THREADS) pool_acc[c] = 0.f;
        __syncthreads();
    }
    const long long i = static_cast<long long>(blockIdx.x) * DW_THREADS + threadIdx.x;
    if (i < items_per_image) {
        const int QT = (Q + TW - 1) / TW;
        const int v = static_cast<int>(i % cv);
        long long t = i / cv;
        const int qt = static_cast<int>(t % QT);
        const int p = static_cast<int>(t / QT);
        const int q0 = qt * TW;

        float acc[TW][8];
        {
            float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (bias) {
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + v * 8));
                const __half2* hb = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __half22float2(hb[k]);
                    b[2 * k] = f.x;
                    b[2 * k + 1] = f.y;
                }
            }
#pragma unroll
            for (int j = 0; j < TW; ++j)
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[j][k] = b[k];
        }

        constexpr int L = (TW - 1) * SW + S;       // input columns one kernel row of the strip touches
        const int iw0 = q0 * SW - pw;
        const __half* ximg = x + n * H * W * ldx + v * 8;
        for (int r = 0; r < R; ++r) {
            const int h = p * sh - ph + r;
            if (h < 0 || h >= H) continue;
            const __half* xrow = ximg + static_cast<long long>(h) * W * ldx;
            const __half* wrow = w + static_cast<long long>(r) * S * C + v * 8;
            float wf[S][8];
#pragma unroll
            for (int s2 = 0; s2 < S; ++s2) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + static_cast<long long>(s2) * C));
                const __half2* hw = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __half22float2(hw[k]);
                    wf[s2][2 * k] = f.x;
                    wf[s2][2 * k + 1] = f.y;
                }
            }
#pragma unroll
            for (int l = 0; l < L; ++l) {
                const int ww = iw0 + l;
                float xf[8];
                if (ww >= 0 && ww < W) {
                    const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xrow + static_cast<long long>(ww) * ldx));
                    const __half2* hx = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __half22float2(hx[k]);
                        xf[2 * k] = f.x;
                        xf[2 * k + 1] = f.y;
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) xf[k] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < TW; ++j) {
                    constexpr int dummy = 0;
                    (void)dummy;
                    const int s2 = l - j * SW;          // compile-time after unrolling
                    if (s2 >= 0 && s2 < S) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) acc[j][k] = fmaf(xf[k], wf[s2][k], acc[j][k]);
                    }
                }
            }
        }

        float psum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < TW; ++j) {
            const int q = q0 + j;
            if (q < Q) {
                __align__(16) __half2 o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    o[k] = __floats2half2_rn(act_f(acc[j][2 * k], act), act_f(acc[j][2 * k + 1], act));
                    if (pool_sums) {
                        const float2 f = __half22float2(o[k]);
                        psum[2 * k] += f.x;
                        psum[2 * k + 1] += f.y;
                    }
                }
                *reinterpret_cast<uint4*>(y + ((n * P + p) * Q + q) * ldy + v * 8) = *reinterpret_cast<uint4*>(o);
            }
        }
        if (pool_sums) {
#pragma unroll
            for (int k = 0; k < 8; ++k) atomicAdd(&pool_acc[v * 8 + k], psum[k]);
        }
    }
    if (pool_sums) {
        __syncthreads();
        for (int c = threadIdx.x; c < C; c += DW_THREADS) {
            const float sum = pool_acc[c];
            if (sum != 0.f) atomicAdd(pool_sums + n * C + c, sum);
        }
    }
}


// Tiled path (the default for square 3/5/7-tap kernels, stride 1 or 2, no dilation): a block stages the input halo
// tile of TH x TWB output pixels x 64 channels in shared memory with 16-byte async copies (out-of-image taps are
// zero-filled by the copy), so every input byte is fetched from L2 about once instead of once per kernel row; each
// thread then produces a strip of 8 output columns for 8 channels from shared memory, with one kernel row of weights
// and the 64 fp32 accumulators in registers. Arithmetic: fp16x2 FMAs within a kernel row, fp32 across rows, as the
// reference's dwconv2 does for the same kernel sizes; every other shape takes the fp32 paths below.
static constexpr int DWT_CBV = 8;        // channel vectors (of 8 channels) per block
static constexpr int DWT_TW = 8;         // output columns per thread
static constexpr int DWT_STRIPS = DW_THREADS / DWT_CBV;   // 16 strips per block

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}

// ACT: activation known at compile time (0 none, 1 relu, 3 silu) or -1 = use the run-time code.
template <int S, int SW, int ACT>
__global__ void __launch_bounds__(DW_THREADS)
dwconv_tile_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const __half* __restrict__ bias,
                   __half* __restrict__ y, float* __restrict__ pool_sums, int H, int W, int C, int R, int P, int Q,
                   int sh, int ph, int pw, long long ldx, long long ldy, int act, int strips_x, int tiles_x,
                   int tiles_y) {
    extern __shared__ __align__(16) uint8_t dw_smem[];
    const int cv = C >> 3;
    const int TH = DWT_STRIPS / strips_x;                 // output rows per block
    const int TWB = strips_x * DWT_TW;                    // output columns per block
    const int tile_h = (TH - 1) * sh + R;
    const int tile_w = (TWB - 1) * SW + S;
    float* pool_acc = reinterpret_cast<float*>(dw_smem + static_cast<size_t>(tile_h) * tile_w * DWT_CBV * 16);

    const long long n = blockIdx.y;
    int bid = blockIdx.x;
    const int tx = bid % tiles_x;
    bid /= tiles_x;
    const int ty = bid % tiles_y;
    const int vb = bid / tiles_y;                          // channel-vector block
    const int p0 = ty * TH, q0 = tx * TWB;
    const int h0 = p0 * sh - ph, w0 = q0 * SW - pw;
    const int v0 = vb * DWT_CBV;

    if (pool_sums && threadIdx.x < DWT_CBV * 8) pool_acc[threadIdx.x] = 0.f;

    // stage the halo tile: [tile_h][tile_w][DWT_CBV] vectors of 16 bytes
    const __half* ximg = x + n * H * W * ldx;
    const uint32_t smem0 = smem_u32(dw_smem);
    const int total = tile_h * tile_w * DWT_CBV;
    for (int idx = threadIdx.x; idx < total; idx += DW_THREADS) {
        const int vv = idx % DWT_CBV;
        const int px = idx / DWT_CBV;
        const int cx = px % tile_w, cy = px / tile_w;
        const int h = h0 + cy, ww = w0 + cx, v = v0 + vv;
        const bool valid = h >= 0 && h < H && ww >= 0 && ww < W && v < cv;
        const __half* src = valid ? ximg + (static_cast<long long>(h) * W + ww) * ldx + v * 8 : ximg;
        cp_async16_zfill(smem0 + static_cast<uint32_t>(idx) * 16u, src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    const int vv = threadIdx.x % DWT_CBV;
    const int strip = threadIdx.x / DWT_CBV;
    const int sx = strip % strips_x, sy = strip / strips_x;
    const int v = v0 + vv;
    const int p = p0 + sy, qs = q0 + sx * DWT_TW;
    const bool active = v < cv && p < P && qs < Q;
    if (active) {
        // fp32 accumulators as packed pairs
        unsigned long long acc[DWT_TW][4];
        {
            unsigned long long b2[4] = {0ull, 0ull, 0ull, 0ull};
            if (bias) {
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + v * 8));
                b2[0] = h2_to_f2(bv.x); b2[1] = h2_to_f2(bv.y); b2[2] = h2_to_f2(bv.z); b2[3] = h2_to_f2(bv.w);
            }
#pragma unroll
            for (int j = 0; j < DWT_TW; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[j][k] = b2[k];
        }
        // Arithmetic of the reference's dwconv2 (classification/fast/csrc/r3.cu:354-415, its default mode): within one
        // kernel row the taps are accumulated with fp16x2 FMAs starting from zero, the row sums are added in fp32.
        // No fp16->fp32 conversion of inputs or weights is needed, which is what made the fp32 version issue-bound.
        constexpr int L = (DWT_TW - 1) * SW + S;
        for (int r = 0; r < R; ++r) {
            const __half* wrow = w + static_cast<long long>(r) * S * C + v * 8;
            uint4 wr[S];
#pragma unroll
            for (int s2 = 0; s2 < S; ++s2)
                wr[s2] = __ldg(reinterpret_cast<const uint4*>(wrow + static_cast<long long>(s2) * C));
            __half2 racc[DWT_TW][4];
#pragma unroll
            for (int j = 0; j < DWT_TW; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k) racc[j][k] = __float2half2_rn(0.f);
            // row (sy*sh + r) of the tile, columns sx*8*SW .. + L
            const uint32_t row_addr =
                smem0 + (static_cast<uint32_t>((sy * sh + r) * tile_w + sx * DWT_TW * SW) * DWT_CBV + vv) * 16u;
#pragma unroll
            for (int l = 0; l < L; ++l) {
                const uint4 xv = lds128(row_addr + static_cast<uint32_t>(l * DWT_CBV) * 16u);
                const __half2* hx = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                for (int j = 0; j < DWT_TW; ++j) {
                    const int s2 = l - j * SW;          // compile-time after unrolling
                    if (s2 >= 0 && s2 < S) {
                        const __half2* hw = reinterpret_cast<const __half2*>(&wr[s2]);
#pragma unroll
                        for (int k = 0; k < 4; ++k) racc[j][k] = __hfma2(hx[k], hw[k], racc[j][k]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < DWT_TW; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    acc[j][k] = f2_add(acc[j][k], h2_to_f2(*reinterpret_cast<const uint32_t*>(&racc[j][k])));
        }
        float psum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < DWT_TW; ++j) {
            const int q = qs + j;
            if (q < Q) {
                __align__(16) __half2 o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    // the sum is rounded to fp16 first; relu acts on the fp16 pair, other activations are evaluated
                    // in fp32 on the rounded value and rounded again (reference: r3.cu:404-413)
                    const uint32_t hv = f2_to_h2(acc[j][k]);
                    o[k] = *reinterpret_cast<const __half2*>(&hv);
                    if (ACT == 1) {
                        o[k] = __hmax2(o[k], __float2half2_rn(0.f));
                    } else if (ACT != 0) {
                        const float2 f = __half22float2(o[k]);
                        if (ACT == 3) {      // SiLU on the pair: packed multiplies, ex2 / rcp per element (no IEEE division)
                            const uint32_t sv = f2_to_h2(f2_silu(f2_pack(__float_as_uint(f.x), __float_as_uint(f.y))));
                            o[k] = *reinterpret_cast<const __half2*>(&sv);
                        }
                        else o[k] = __floats2half2_rn(act_f(f.x, act), act_f(f.y, act));
                    }
                    if (pool_sums) {
                        const float2 f = __half22float2(o[k]);
                        psum[2 * k] += f.x;
                        psum[2 * k + 1] += f.y;
                    }
                }
                *reinterpret_cast<uint4*>(y + ((n * P + p) * Q + q) * ldy + v * 8) = *reinterpret_cast<uint4*>(o);
            }
        }
        if (pool_sums) {
#pragma unroll
            for (int k = 0; k < 8; ++k) atomicAdd(&pool_acc[vv * 8 + k], psum[k]);
        }
    }
    if (pool_sums) {
        __syncthreads();
        if (threadIdx.x < DWT_CBV * 8) {
            const int c = v0 * 8 + threadIdx.x;
            const float sum = pool_acc[threadIdx.x];
            if (c < C && sum != 0.f) atomicAdd(pool_sums + n * C + c, sum);
        }
    }
}

template <int S, int SW, int ACT>
static int launch_dw_tile_act(const __half* xp, const __half* wp, const __half* bp, __half* yp, float* pool_sums, int N, int H,
                          int W, int C, int R, int P, int Q, int sh, int ph, int pw, long long ldx, long long ldy, int act,
                          cudaStream_t st) {
    const int cv = C >> 3;
    const int strips_x = Q > DWT_TW ? 2 : 1;
    const int TH = DWT_STRIPS / strips_x, TWB = strips_x * DWT_TW;
    const int tile_h = (TH - 1) * sh + R, tile_w = (TWB - 1) * SW + S;
    const size_t smem = static_cast<size_t>(tile_h) * tile_w * DWT_CBV * 16 + DWT_CBV * 8 * sizeof(float);
    if (smem > 200 * 1024) return -1;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(dwconv_tile_kernel<S, SW, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
            cudaSuccess)
            return FVM_ERR_SETUP;
        attr_set = true;
    }
    const int tiles_x = (Q + TWB - 1) / TWB, tiles_y = (P + TH - 1) / TH, vblocks = (cv + DWT_CBV - 1) / DWT_CBV;
    const long long bx = static_cast<long long>(tiles_x) * tiles_y * vblocks;
    if (bx > 0x7fffffffll) return FVM_ERR_ARG;
    dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(N));
    dwconv_tile_kernel<S, SW, ACT><<<grid, DW_THREADS, smem, st>>>(xp, wp, bp, yp, pool_sums, H, W, C, R, P, Q, sh, ph, pw, ldx,
                                                              ldy, act, strips_x, tiles_x, tiles_y);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}

}  // namespace fvm

using namespace fvm;

extern "C" int fvm_dwconv_f16(const void* x, const void* w_rsc, const void* bias, void* y, float* pool_sums, int N,
                              int H, int W, int C, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                              long long ldx, long long ldy, int act, void* stream) {
    if (!x || !w_rsc || !y || N <= 0 || N > 65535 || H <= 0 || W <= 0 || C <= 0 || (C & 7) || R <= 0 || S <= 0 ||
        sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || ph < 0 || pw < 0 || (ldx & 7) || (ldy & 7) || ldx < C || ldy < C ||
        act < 0 || act > 6)
        return FVM_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w_rsc) & 15) ||
        (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(bias) & 15))
        return FVM_ERR_ARG;
    if (pool_sums && C > DW_MAX_POOL_C) return FVM_ERR_ARG;
    const int P = (H + 2 * ph - dh * (R - 1) - 1) / sh + 1;
    const int Q = (W + 2 * pw - dw * (S - 1) - 1) / sw + 1;
    if (P <= 0 || Q <= 0) return FVM_ERR_ARG;
    const int cv = C >> 3;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xp = static_cast<const __half*>(x);
    const __half* wp = static_cast<const __half*>(w_rsc);
    const __half* bp = static_cast<const __half*>(bias);
    __half* yp = static_cast<__half*>(y);
    const size_t smem = pool_sums ? static_cast<size_t>(C) * sizeof(float) : 0;
    // Fast path: square 3/5/7 kernels, stride 1 or 2 (same in both directions), no dilation. Strips of 8 outputs on
    // wide maps, 4 on narrow ones (the grid must still cover the machine a few times over).
    if (R == S && (S == 3 || S == 5 || S == 7) && dh == 1 && dw == 1 && sh == sw && (sw == 1 || sw == 2) && Q >= 4) {
        int rc = -1;
        if (S == 3) rc = sw == 1 ? launch_dw_tile<3, 1>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st)
                                 : launch_dw_tile<3, 2>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st);
        else if (S == 5) rc = sw == 1 ? launch_dw_tile<5, 1>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st)
                                      : launch_dw_tile<5, 2>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st);
        else rc = sw == 1 ? launch_dw_tile<7, 1>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st)
                          : launch_dw_tile<7, 2>(xp, wp, bp, yp, pool_sums, N, H, W, C, R, P, Q, sh, ph, pw, ldx, ldy, act, st);
        if (rc >= 0) return rc;      // -1: the tile does not fit shared memory, use the register path below
    }
    if (R == S && (S == 3 || S == 5 || S == 7) && dh == 1 && dw == 1 && sh == sw && (sw == 1 || sw == 2)) {
        const long long work8 = static_cast<long long>(N) * P * ((Q + 7) / 8) * cv;
        const int TWF = (Q >= 24 && work8 >= 148ll * 4 * DW_THREADS && S < 7) ? 8 : 4;
        const int QTF = (Q + TWF - 1) / TWF;
        const long long itemsF = static_cast<long long>(P) * QTF * cv;
        const long long bxF = (itemsF + DW_THREADS - 1) / DW_THREADS;
        if (bxF > 0x7fffffffll) return FVM_ERR_ARG;
        dim3 gridF(static_cast<unsigned>(bxF), static_cast<unsigned>(N));
#define DWF_GO(SV, SWV, TWV)                                                                                       \
    dwconv_fast_kernel<SV, SWV, TWV><<<gridF, DW_THREADS, smem, st>>>(xp, wp, bp, yp, pool_sums, H, W, C, R, P, Q, sh, \
                                                                      ph, pw, ldx, ldy, act, itemsF)
#define DWF_S(SV)                                   \
    do {                                            \
        if (sw == 1) {                              \
            if (TWF == 8) DWF_GO(SV, 1, 8);         \
            else DWF_GO(SV, 1, 4);                  \
        } else {                                    \
            if (TWF == 8) DWF_GO(SV, 2, 8);         \
            else DWF_GO(SV, 2, 4);                  \
        }                                           \
    } while (0)
        if (S == 3) DWF_S(3);
        else if (S == 5) DWF_S(5);
        else DWF_S(7);
#undef DWF_S
#undef DWF_GO
        count_launch();
        return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
    }
    // wide strips where rows are long; narrow ones on small maps so that the grid still fills the machine
    const int TW = Q >= 32 ? 4 : (Q >= 12 ? 2 : 1);
    const int QT = (Q + TW - 1) / TW;
    const long long items = static_cast<long long>(P) * QT * cv;
    const long long bx = (items + DW_THREADS - 1) / DW_THREADS;
    if (bx > 0x7fffffffll) return FVM_ERR_ARG;
    dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(N));
#define DW_GO(TWV)                                                                                                    \
    dwconv_kernel<TWV><<<grid, DW_THREADS, smem, st>>>(xp, wp, bp, yp, pool_sums, H, W, C, R, S, P, Q, sh, sw, ph, pw, \
                                                       dh, dw, ldx, ldy, act, items)
    if (TW == 4) DW_GO(4);
    else if (TW == 2) DW_GO(2);
    else DW_GO(1);
#undef DW_GO
    count_launch();
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}
