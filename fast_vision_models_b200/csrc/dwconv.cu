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
    // wide strips where rows are long; narrow ones on small maps so that the grid still fills the machine
    const int TW = Q >= 32 ? 4 : (Q >= 12 ? 2 : 1);
    const int QT = (Q + TW - 1) / TW;
    const long long items = static_cast<long long>(P) * QT * cv;
    const long long bx = (items + DW_THREADS - 1) / DW_THREADS;
    if (bx > 0x7fffffffll) return FVM_ERR_ARG;
    dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(N));
    const size_t smem = pool_sums ? static_cast<size_t>(C) * sizeof(float) : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xp = static_cast<const __half*>(x);
    const __half* wp = static_cast<const __half*>(w_rsc);
    const __half* bp = static_cast<const __half*>(bias);
    __half* yp = static_cast<__half*>(y);
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
