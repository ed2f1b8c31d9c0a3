// HBM-bound NHWC fp16 kernels of the convolutional hot path: layout conversion, pooling, global average pool,
// squeeze-excite gate and scale, channels-last LayerNorm, elementwise epilogues, bilinear resize and fused
// upsample+argmax. All of them move 16 bytes (8 channels) per thread per access, accumulate in fp32 and round once.
#include <cstdint>
#include <mutex>

#include "fvm_internal.h"
#include "ptx_sm100.cuh"

namespace fvm {

union V8 {
    uint4 u;
    __half2 h2[4];
    __half h[8];
};

__device__ __forceinline__ uint4 ldg16(const __half* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void stg16(__half* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

__device__ __forceinline__ void to_f8(const uint4& u, float (&f)[8]) {
    V8 v;
    v.u = u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(v.h2[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 from_f8(const float (&f)[8]) {
    V8 v;
#pragma unroll
    for (int i = 0; i < 4; ++i) v.h2[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v.u;
}

static inline int blocks_for(long long items, int threads) {
    long long b = (items + threads - 1) / threads;
    if (b < 1) b = 1;
    if (b > 0x7fffffffll) b = 0x7fffffffll;
    return static_cast<int>(b);
}

// ------------------------------------------------------------------------------------------- input fp32 NCHW -> NHWC8
// y[n,h,w,c] = c < C ? half(x[n,c,h,w]) : 0   (reference: classification/fast/csrc/fused_conv.cu:597-606)
__device__ __forceinline__ float in_f32(float v) { return v; }
__device__ __forceinline__ float in_f32(__half v) { return __half2float(v); }

// T = float or __half: the reference's kernel is a template over both input types (fused_conv.cu:597-620).
template <class T>
__global__ void input_nhwc8_kernel(const T* __restrict__ x, __half* __restrict__ y, int C, long long HW,
                                   long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / HW;
    const long long hw = i - n * HW;
    const T* src = x + n * C * HW + hw;
    float f[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) f[c] = c < C ? in_f32(__ldg(src + c * HW)) : 0.f;
    stg16(y + i * 8, from_f8(f));
}

// The same conversion into two column-parity planes per image row: y[n][h][w & 1][w >> 1][c] (W even). A stride-2
// convolution then reads consecutive output columns from consecutive plane columns (see the stem mode of the conv kernel).
template <class T>
__global__ void input_nhwc8_split_kernel(const T* __restrict__ x, __half* __restrict__ y, int C, int H, int W) {
    // blockIdx.x = image row (n * H + h), blockIdx.y = chunk of columns: one division per thread
    const int w = blockIdx.y * blockDim.x + threadIdx.x;
    if (w >= W) return;
    const long long HW = static_cast<long long>(H) * W;
    const long long nh = blockIdx.x;
    const long long n = nh / H;
    const long long hrow = nh - n * H;
    const T* src = x + n * C * HW + hrow * W + w;
    float f[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) f[c] = c < C ? in_f32(__ldg(src + c * HW)) : 0.f;
    const long long o = nh * W + static_cast<long long>(w & 1) * (W >> 1) + (w >> 1);
    stg16(y + o * 8, from_f8(f));
}

// ------------------------------------------------------------------------------------------- max / avg pool
// reference: maxpool_nhwc8 (fused_conv.cu:338-356): -inf padding, half2 max over in-image taps only.
__global__ void maxpool_kernel(const __half* __restrict__ x, __half* __restrict__ y, int H, int W, int C, int kh, int kw,
                               int sh, int sw, int ph, int pw, int P, int Q, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    long long t = i / cv;
    const int q = static_cast<int>(t % Q);
    t /= Q;
    const int pp = static_cast<int>(t % P);
    const long long n = t / P;
    V8 m;
    const __half2 ninf = __half2half2(__ushort_as_half(0xfc00));
#pragma unroll
    for (int j = 0; j < 4; ++j) m.h2[j] = ninf;
    const int h0 = pp * sh - ph, w0 = q * sw - pw;
    for (int r = 0; r < kh; ++r) {
        const int h = h0 + r;
        if (h < 0 || h >= H) continue;
        for (int s = 0; s < kw; ++s) {
            const int w = w0 + s;
            if (w < 0 || w >= W) continue;
            V8 a;
            a.u = ldg16(x + ((n * H + h) * W + w) * C + v * 8);
#pragma unroll
            for (int j = 0; j < 4; ++j) m.h2[j] = __hmax2(m.h2[j], a.h2[j]);
        }
    }
    stg16(y + i * 8, m.u);
}

// reference: avgpool_nhwc8 (fused_conv.cu:556-582): fp32 sum over in-image taps, PyTorch divisor rule.
__global__ void avgpool_kernel(const __half* __restrict__ x, __half* __restrict__ y, int H, int W, int C, int kh, int kw,
                               int sh, int sw, int ph, int pw, int P, int Q, int include_pad, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    long long t = i / cv;
    const int q = static_cast<int>(t % Q);
    t /= Q;
    const int pp = static_cast<int>(t % P);
    const long long n = t / P;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int h0 = pp * sh - ph, w0 = q * sw - pw;
    int cnt = 0;
    for (int r = 0; r < kh; ++r) {
        const int h = h0 + r;
        if (h < 0 || h >= H) continue;
        for (int s = 0; s < kw; ++s) {
            const int w = w0 + s;
            if (w < 0 || w >= W) continue;
            float f[8];
            to_f8(ldg16(x + ((n * H + h) * W + w) * C + v * 8), f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += f[j];
            ++cnt;
        }
    }
    int div;
    if (include_pad) {
        const int hend = min(h0 + kh, H + ph), wend = min(w0 + kw, W + pw);
        div = (hend - h0) * (wend - w0);
    } else {
        div = max(cnt, 1);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = acc[j] / static_cast<float>(div);
    stg16(y + i * 8, from_f8(acc));
}

// ------------------------------------------------------------------------------------------- global average pool
// Stage 1: block (32 channel-vectors x 8 pixel rows); grid (ceil(cv/32), splits, N). Each thread sums its pixels of
// one split in a fixed order, the 8 rows are combined in a fixed order in shared memory -> partial[n][split][c].
// Stage 2 sums the splits in order and scales. Summation order is therefore fixed: results are deterministic.
static constexpr int GAP_VX = 32, GAP_RY = 8;

// With a single split (maps of up to 64 pixels) stage 2 has nothing to add: `y_direct` != nullptr makes stage 1 write
// the fp16 means itself (same sums, same order, same rounding as the two-stage path) and stage 2 is not launched.
__global__ void gap_partial_kernel(const __half* __restrict__ x, float* __restrict__ partial, int HW, int C,
                                   long long ldx, int splits, int chunk, __half* __restrict__ y_direct, float inv_hw) {
    __shared__ float red[GAP_RY][GAP_VX][8];
    const int cv = C >> 3;
    const int v = blockIdx.x * GAP_VX + threadIdx.x;
    const int split = blockIdx.y;
    const long long n = blockIdx.z;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (v < cv) {
        const int p0 = split * chunk;
        const int p1 = min(HW, p0 + chunk);
        const __half* base = x + n * HW * ldx + v * 8;
        for (int px = p0 + threadIdx.y; px < p1; px += GAP_RY) {
            float f[8];
            to_f8(ldg16(base + px * ldx), f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x][j] = acc[j];
    __syncthreads();
    if (threadIdx.y == 0 && v < cv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float s = red[0][threadIdx.x][j];
            for (int r = 1; r < GAP_RY; ++r) s += red[r][threadIdx.x][j];
            if (y_direct) y_direct[n * C + v * 8 + j] = __float2half_rn(s * inv_hw);
            else partial[(n * splits + split) * C + v * 8 + j] = s;
        }
    }
}

__global__ void gap_final_kernel(const float* __restrict__ partial, __half* __restrict__ y, int C, int splits,
                                 float inv_hw, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / C;
    const int c = static_cast<int>(i - n * C);
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partial[(n * splits + k) * C + c];
    y[i] = __float2half_rn(s * inv_hw);
}

static int gap_splits(int N, int HW, int C, int sms) {
    const int cvb = ((C >> 3) + GAP_VX - 1) / GAP_VX;
    const long long base_blocks = static_cast<long long>(N) * cvb;
    long long want = (4ll * sms + base_blocks - 1) / base_blocks;
    long long max_splits = (HW + 63) / 64;   // at least 64 pixels (8 per thread) per split
    if (want > max_splits) want = max_splits;
    if (want < 1) want = 1;
    if (want > 1024) want = 1024;
    return static_cast<int>(want);
}

// ------------------------------------------------------------------------------------------- squeeze-excite gate
// gridDim.y blocks per image: each computes h = half(act(W1 g + b1)) (warp per output, lanes stride over C; the
// squeeze FC is small, so it is recomputed per block rather than exchanged) and its slice of s = half(W2 h + b2)
// (thread per output). Rounding points follow the two conv_fused calls the reference issues on [N,C,1,1] tensors.
__global__ void se_gate_kernel(const void* __restrict__ g_in, const __half* __restrict__ w1,
                               const __half* __restrict__ b1, const __half* __restrict__ w2,
                               const __half* __restrict__ b2, __half* __restrict__ s_out, int C, int Cs, int act,
                               float mean_scale, int slots, int sgroups) {
    extern __shared__ float sm[];
    float* g = sm;          // [C]
    float* h = sm + C;      // [Cs]
    const long long n = blockIdx.x;
    if (mean_scale != 0.f) {
        // fused squeeze: fp32 partial sums [slots][C] of this image times 1 / pixels. The slots are cut into `sgroups`
        // contiguous runs that are summed in parallel (every thread busy, several loads in flight), then the runs are
        // added in order: a fixed summation order, whatever the scheduling.
        const float* gs = static_cast<const float*>(g_in) + n * slots * C;
        float* part = sm + C + Cs;                 // [sgroups][C]
        const int run = (slots + sgroups - 1) / sgroups;
        for (int idx = threadIdx.x; idx < C * sgroups; idx += blockDim.x) {
            const int sg = idx / C, c = idx - sg * C;
            const int k1 = min(slots, (sg + 1) * run);
            float sum = 0.f;
#pragma unroll 8
            for (int k = sg * run; k < k1; ++k) sum += gs[static_cast<long long>(k) * C + c];
            part[idx] = sum;
        }
        __syncthreads();
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            float sum = part[c];
            for (int sg = 1; sg < sgroups; ++sg) sum += part[sg * C + c];
            g[c] = __half2float(__float2half_rn(sum * mean_scale));
        }
    } else {
        const __half* gh = static_cast<const __half*>(g_in) + n * C;
        for (int c = threadIdx.x; c < C; c += blockDim.x) g[c] = __half2float(gh[c]);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int cv = C >> 3;
    // FC1: a warp takes two rows of W1 at a time (eight 16-byte loads in flight per lane: the rows come from L2 and the
    // loop is bound by that latency, not by arithmetic); each row's products are added in the same order as one by one
    for (int j = 2 * warp; j < Cs; j += 2 * nwarps) {
        const bool two = j + 1 < Cs;
        const __half* row0 = w1 + static_cast<long long>(j) * C;
        const __half* row1 = row0 + (two ? C : 0);
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 4
        for (int v = lane; v < cv; v += 32) {
            float f0[8], f1[8];
            to_f8(ldg16(row0 + v * 8), f0);
            to_f8(ldg16(row1 + v * 8), f1);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                acc0 = fmaf(f0[k], g[v * 8 + k], acc0);
                acc1 = fmaf(f1[k], g[v * 8 + k], acc1);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, o);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
        }
        if (lane == 0) {
            if (b1) acc0 += __half2float(b1[j]);
            h[j] = __half2float(__float2half_rn(act_f(acc0, act)));
            if (two) {
                if (b1) acc1 += __half2float(b1[j + 1]);
                h[j + 1] = __half2float(__float2half_rn(act_f(acc1, act)));
            }
        }
    }
    __syncthreads();
    // FC2: one output per thread and pass; the row of W2 (Cs halves) is fetched with all its loads in flight
    const int sv = Cs >> 3;
    const int per = (C + gridDim.y - 1) / gridDim.y, c_end = min(C, static_cast<int>(blockIdx.y + 1) * per);
    for (int c = blockIdx.y * per + threadIdx.x; c < c_end; c += blockDim.x) {
        const __half* row = w2 + static_cast<long long>(c) * Cs;
        float acc = 0.f;
        for (int v0 = 0; v0 < sv; v0 += 8) {
            uint4 q[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (v0 + u < sv) q[u] = ldg16(row + (v0 + u) * 8);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (v0 + u < sv) {
                    float f[8];
                    to_f8(q[u], f);
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc = fmaf(f[k], h[(v0 + u) * 8 + k], acc);
                }
            }
        }
        if (b2) acc += __half2float(b2[c]);
        s_out[n * C + c] = __float2half_rn(acc);
    }
}

// y = x * sigmoid(s[n,c]) -- reference se_scale_k (classification/fast/csrc/r3.cu:302-317): sigmoid in fp32, rounded
// to fp16, fp16 multiply.
__global__ void se_scale_kernel(const __half* __restrict__ x, const __half* __restrict__ s, __half* __restrict__ y,
                                int HW, int C, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    const long long n = i / (static_cast<long long>(cv) * HW);
    V8 a, g, o;
    a.u = ldg16(x + i * 8);
    g.u = ldg16(s + n * C + v * 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 t = __half22float2(g.h2[j]);
        // sigmoid as rcp(1 + 2^(-t log2 e)) with the approximate reciprocal (1-2 fp32 ulp, far inside the fp16 rounding
        // that follows): the IEEE division made this kernel issue-bound
        __half2 sg = __floats2half2_rn(__fdividef(1.f, 1.f + __expf(-t.x)), __fdividef(1.f, 1.f + __expf(-t.y)));
        o.h2[j] = __hmul2(a.h2[j], sg);
    }
    stg16(y + i * 8, o.u);
}

// Squeeze-excite gate folded into the weights of the 1x1 conv that follows: out[n][k][c] = half(w[k][c] * half(sigmoid(s[n][c])))
// -- the same rounded gate as se_scale_kernel multiplies the activations with (reference: r3.cu:312-315), applied to
// the other operand of the products instead, so that the scaled activation tensor is never written or re-read.
__global__ void gate_weights_kernel(const __half* __restrict__ w, const __half* __restrict__ s, __half* __restrict__ out,
                                    int K, int C, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;     // one 8-channel vector
    if (i >= total) return;
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    const long long t = i / cv;
    const int k = static_cast<int>(t % K);
    const long long n = t / K;
    V8 a, g, o;
    a.u = ldg16(w + (static_cast<long long>(k) * C + v * 8));
    g.u = ldg16(s + n * C + v * 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(g.h2[j]);
        const __half2 sg = __floats2half2_rn(__fdividef(1.f, 1.f + __expf(-f.x)), __fdividef(1.f, 1.f + __expf(-f.y)));
        o.h2[j] = __hmul2(a.h2[j], sg);
    }
    stg16(out + i * 8, o.u);
}

// ------------------------------------------------------------------------------------------- channels-last LayerNorm
// G lanes cooperate on one row (G = 4, 8, 16 or 32) and each lane holds VPL 16-byte vectors of it, G * VPL being the
// smallest cover of the row's C / 8 vectors (C = 96: 4 lanes x 3 vectors, every lane busy). A lane group normalises
// RPG rows at a time: the loads of all of them are issued before the first reduction, which is what keeps enough bytes
// in flight per SM for an HBM-bound kernel. Two-pass fp32 statistics (mean, then sum of squared deviations), fp32
// affine, one rounding; gamma / beta are loaded once per thread.
template <int G, int VPL, int RPG>
__global__ void __launch_bounds__(256)
layernorm_cl_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma, const __half* __restrict__ beta,
                    __half* __restrict__ y, long long rows, int C, float eps, long long ldx, long long ldy) {
    constexpr int GROUPS = 32 / G;
    const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / G, gl = lane % G;
    const long long group = (static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp_in_block) * GROUPS + sub;
    const long long row0 = group * RPG;
    const int cv = C >> 3;
    float f[RPG][VPL][8];
#pragma unroll
    for (int r = 0; r < RPG; ++r)
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
            const int v = gl + k * G;
            if (row0 + r < rows && v < cv) {
                to_f8(ldg16(x + (row0 + r) * ldx + v * 8), f[r][k]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[r][k][j] = 0.f;
            }
        }
    float gm[VPL][8], bt[VPL][8];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int v = gl + k * G;
#pragma unroll
        for (int j = 0; j < 8; ++j) { gm[k][j] = 1.f; bt[k][j] = 0.f; }
        if (v < cv) {
            if (gamma) to_f8(ldg16(gamma + v * 8), gm[k]);
            if (beta) to_f8(ldg16(beta + v * 8), bt[k]);
        }
    }
    const float inv_c = 1.f / static_cast<float>(C);
#pragma unroll
    for (int r = 0; r < RPG; ++r) {
        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < VPL; ++k)
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += f[r][k][j];
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum * inv_c;
        float sq = 0.f;
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
            if (gl + k * G < cv) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float d = f[r][k][j] - mean;
                    sq += d * d;
                }
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float rstd = rsqrtf(sq * inv_c + eps);
        if (row0 + r < rows) {
#pragma unroll
            for (int k = 0; k < VPL; ++k) {
                const int v = gl + k * G;
                if (v < cv) {
                    float o[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = (f[r][k][j] - mean) * rstd * gm[k][j] + bt[k][j];
                    stg16(y + (row0 + r) * ldy + v * 8, from_f8(o));
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------- elementwise epilogues
// reference: bias_act_h (segmentation/fast/csrc/seg_kernels.cu:107-119)
__global__ void bias_act_kernel(__half* __restrict__ y, const __half* __restrict__ bias, const __half* __restrict__ res,
                                int C, int relu, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    float f[8];
    to_f8(*reinterpret_cast<const uint4*>(y + i * 8), f);
    if (bias) {
        float b[8];
        to_f8(ldg16(bias + v * 8), b);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += b[j];
    }
    if (res) {
        float r[8];
        to_f8(ldg16(res + i * 8), r);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += r[j];
    }
    if (relu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
    }
    stg16(y + i * 8, from_f8(f));
}

// reference: affine_act_k (classification/fast/csrc/fused_conv.cu:310-321)
__global__ void affine_act_kernel(const __half* __restrict__ x, const float* __restrict__ scale,
                                  const float* __restrict__ shift, __half* __restrict__ y, int C, long long ldx,
                                  long long ldy, int act, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    const long long px = i / cv;
    float f[8];
    to_f8(ldg16(x + px * ldx + v * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = act_f(f[j] * __ldg(scale + v * 8 + j) + __ldg(shift + v * 8 + j), act);
    stg16(y + px * ldy + v * 8, from_f8(f));
}

__global__ void add_act_kernel(const __half* __restrict__ a, const __half* __restrict__ b, __half* __restrict__ y,
                               int act, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float fa[8], fb[8];
    to_f8(ldg16(a + i * 8), fa);
    to_f8(ldg16(b + i * 8), fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) fa[j] = act_f(fa[j] + fb[j], act);
    stg16(y + i * 8, from_f8(fa));
}

// ------------------------------------------------------------------------------------------- bilinear resize
// PyTorch index math (reference: bilin_k, segmentation/fast/csrc/segx_ops.cu:62-111).
__device__ __forceinline__ void src_index(int i, float scale, int align, int in, int& i0, int& i1, float& l) {
    float f = align ? i * scale : fmaxf((i + 0.5f) * scale - 0.5f, 0.f);
    i0 = min(static_cast<int>(f), in - 1);
    i1 = i0 + (i0 < in - 1 ? 1 : 0);
    l = f - i0;
}

__global__ void bilinear_kernel(const __half* __restrict__ x, const __half* __restrict__ base, __half* __restrict__ y,
                                int h, int w, int C, int H, int W, int align, float sch, float scw, int relu,
                                long long ldx, long long ldy, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    long long t = i / cv;
    const int ox = static_cast<int>(t % W);
    t /= W;
    const int oy = static_cast<int>(t % H);
    const long long n = t / H;
    int y0, y1, x0, x1;
    float ly, lx;
    src_index(oy, sch, align, h, y0, y1, ly);
    src_index(ox, scw, align, w, x0, x1, lx);
    const float hy = 1.f - ly, hx = 1.f - lx;
    const __half* img = x + n * h * w * ldx + v * 8;
    float a[8], b[8], c[8], d[8], o[8];
    to_f8(ldg16(img + (static_cast<long long>(y0) * w + x0) * ldx), a);
    to_f8(ldg16(img + (static_cast<long long>(y0) * w + x1) * ldx), b);
    to_f8(ldg16(img + (static_cast<long long>(y1) * w + x0) * ldx), c);
    to_f8(ldg16(img + (static_cast<long long>(y1) * w + x1) * ldx), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = hy * (hx * a[j] + lx * b[j]) + ly * (hx * c[j] + lx * d[j]);
    const long long opix = (n * H + oy) * W + ox;
    if (base) {
        // the interpolated value is rounded to fp16 first, then added in fp32 (segx_ops.cu:102-105)
        float bb[8];
        to_f8(ldg16(base + opix * ldy + v * 8), bb);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            o[j] = __half2float(__float2half_rn(o[j])) + bb[j];
            if (relu) o[j] = fmaxf(o[j], 0.f);
        }
    }
    stg16(y + opix * ldy + v * 8, from_f8(o));
}

// Fused bilinear upsample + argmax over channels; first maximum wins; scores are not rounded between the lerp and
// the comparison (reference: up_argmax_h, segmentation/fast/csrc/seg_kernels.cu:11-42).
__global__ void up_argmax_kernel(const __half* __restrict__ s, int32_t* __restrict__ out, int h, int w, int C,
                                 long long ld, int H, int W, int align, float sch, float scw, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int ox = static_cast<int>(i % W);
    long long t = i / W;
    const int oy = static_cast<int>(t % H);
    const long long n = t / H;
    int y0, y1, x0, x1;
    float ly, lx;
    src_index(oy, sch, align, h, y0, y1, ly);
    src_index(ox, scw, align, w, x0, x1, lx);
    const float hy = 1.f - ly, hx = 1.f - lx;
    const __half* img = s + n * h * w * ld;
    const __half* pa = img + (static_cast<long long>(y0) * w + x0) * ld;
    const __half* pb = img + (static_cast<long long>(y0) * w + x1) * ld;
    const __half* pc = img + (static_cast<long long>(y1) * w + x0) * ld;
    const __half* pd = img + (static_cast<long long>(y1) * w + x1) * ld;
    float best = -INFINITY;
    int arg = 0;
    for (int c0 = 0; c0 < C; c0 += 8) {
        float a[8], b[8], c[8], d[8];
        to_f8(ldg16(pa + c0), a);
        to_f8(ldg16(pb + c0), b);
        to_f8(ldg16(pc + c0), c);
        to_f8(ldg16(pd + c0), d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float val = hy * (hx * a[j] + lx * b[j]) + ly * (hx * c[j] + lx * d[j]);
            if (c0 + j < C && val > best) {
                best = val;
                arg = c0 + j;
            }
        }
    }
    out[i] = arg;
}

// The same for an upsample by a power-of-two factor SF without corner alignment (the DeepLab tail: SF = 8). The SF
// output pixels [g*SF - SF/2, g*SF + SF/2) of a row lie between the same two source columns g - 1 and g, so one thread
// takes such a group: it loads and converts the four source pixels once, interpolates vertically once per channel and
// then only the horizontal lerp and the comparison are per output pixel -- about a fifth of the instructions of the
// per-pixel kernel, which is bound by the FMA pipe. Weights come from the same index function; the sums are formed
// in another order than in up_argmax_kernel (vertical first), so a class map can differ from it where two scores are
// within a rounding error of each other.
template <int SF>
__global__ void up_argmax_group_kernel(const __half* __restrict__ s, int32_t* __restrict__ out, int h, int w, int C,
                                       long long ld, int H, int W, float sch, float scw, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int g = static_cast<int>(i % (w + 1));
    long long t = i / (w + 1);
    const int oy = static_cast<int>(t % H);
    const long long n = t / H;
    const int ox0 = g * SF - SF / 2;
    const int j0 = ox0 < 0 ? -ox0 : 0, j1 = ox0 + SF > W ? W - ox0 : SF;     // valid outputs of this group
    int y0, y1, x0, x1;
    float ly, lx[SF];
    src_index(oy, sch, 0, h, y0, y1, ly);
    {
        float l;
        src_index(ox0 + j0, scw, 0, w, x0, x1, l);
    }
#pragma unroll
    for (int j = 0; j < SF; ++j) {
        int a0, a1;
        src_index(min(max(ox0 + j, 0), W - 1), scw, 0, w, a0, a1, lx[j]);
    }
    const float hy = 1.f - ly;
    const __half* img = s + n * h * w * ld;
    const __half* pa = img + (static_cast<long long>(y0) * w + x0) * ld;
    const __half* pb = img + (static_cast<long long>(y0) * w + x1) * ld;
    const __half* pc = img + (static_cast<long long>(y1) * w + x0) * ld;
    const __half* pd = img + (static_cast<long long>(y1) * w + x1) * ld;
    float best[SF];
    int arg[SF];
#pragma unroll
    for (int j = 0; j < SF; ++j) {
        best[j] = -INFINITY;
        arg[j] = 0;
    }
    for (int c0 = 0; c0 < C; c0 += 8) {
        float a[8], b[8], c[8], d[8];
        to_f8(ldg16(pa + c0), a);
        to_f8(ldg16(pb + c0), b);
        to_f8(ldg16(pc + c0), c);
        to_f8(ldg16(pd + c0), d);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < C) {
                const float va = hy * a[k] + ly * c[k], vb = hy * b[k] + ly * d[k];
#pragma unroll
                for (int j = 0; j < SF; ++j) {
                    const float val = (1.f - lx[j]) * va + lx[j] * vb;
                    if (val > best[j]) {
                        best[j] = val;
                        arg[j] = c0 + k;
                    }
                }
            }
        }
    }
    int32_t* dst = out + (n * H + oy) * W + ox0;
    if (SF >= 4 && j0 == 0 && j1 == SF && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < SF; j += 4) *reinterpret_cast<int4*>(dst + j) = make_int4(arg[j], arg[j + 1], arg[j + 2], arg[j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < SF; ++j)
            if (j >= j0 && j < j1) dst[j] = arg[j];
    }
}

// ------------------------------------------------------------------------------------------- host wrappers
#define FVM_LAUNCH_CHECK()                                                   \
    do {                                                                     \
        count_launch();                                                      \
        return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;  \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace fvm

using namespace fvm;

template <class T>
static int input_nhwc8_launch(const T* x, void* y, int N, int C, int H, int W, void* stream) {
    if (!x || !y || N <= 0 || C <= 0 || C > 8 || H <= 0 || W <= 0 || !aligned16(y)) return FVM_ERR_ARG;
    const long long HW = static_cast<long long>(H) * W, total = HW * N;
    input_nhwc8_kernel<T><<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, static_cast<__half*>(y), C, HW, total);
    FVM_LAUNCH_CHECK();
}

// fp32 images whose rows are whole float4s: a thread converts four neighbouring pixels (three 16-byte loads instead of
// twelve 4-byte ones) and writes two neighbouring pixels into each parity plane.
__global__ void input_nhwc8_split4_kernel(const float* __restrict__ x, __half* __restrict__ y, int C, int H, int W,
                                          long long quads) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= quads) return;
    const int qpr = W >> 2;                       // quads per image row
    const long long nh = i / qpr;                 // n * H + h
    const int w0 = static_cast<int>(i - nh * qpr) * 4;
    const long long HW = static_cast<long long>(H) * W;
    const long long n = nh / H;
    const long long hrow = nh - n * H;
    const float* src = x + n * C * HW + hrow * W + w0;
    float4 v[3];
#pragma unroll
    for (int c = 0; c < 3; ++c) v[c] = c < C ? __ldg(reinterpret_cast<const float4*>(src + c * HW)) : make_float4(0.f, 0.f, 0.f, 0.f);
    float px[4][8];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
#pragma unroll
        for (int c = 0; c < 8; ++c) px[p][c] = 0.f;
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        px[0][c] = v[c].x; px[1][c] = v[c].y; px[2][c] = v[c].z; px[3][c] = v[c].w;
    }
    __half* even = y + (nh * W + (w0 >> 1)) * 8;                 // plane of even columns: positions w0/2, w0/2 + 1
    __half* odd = even + static_cast<long long>(W >> 1) * 8;      // plane of odd columns
    stg16(even, from_f8(px[0]));
    stg16(even + 8, from_f8(px[2]));
    stg16(odd, from_f8(px[1]));
    stg16(odd + 8, from_f8(px[3]));
}

template <class T>
static int input_nhwc8_split_launch(const T* x, void* y, int N, int C, int H, int W, void* stream) {
    if (!x || !y || N <= 0 || C <= 0 || C > 8 || H <= 0 || W <= 0 || (W & 1) || !aligned16(y)) return FVM_ERR_ARG;
    const long long rows = static_cast<long long>(N) * H;
    if (rows > 2147483647ll) return FVM_ERR_ARG;
    if (sizeof(T) == 4 && C <= 3 && (W & 3) == 0 && aligned16(x)) {
        const long long quads = rows * (W >> 2);
        input_nhwc8_split4_kernel<<<blocks_for(quads, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const float*>(x), static_cast<__half*>(y), C, H, W, quads);
        FVM_LAUNCH_CHECK();
    }
    const int tpb = W >= 256 ? 256 : (W >= 128 ? 128 : 64);
    const dim3 grid(static_cast<unsigned>(rows), static_cast<unsigned>((W + tpb - 1) / tpb), 1);
    input_nhwc8_split_kernel<T><<<grid, tpb, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<__half*>(y), C, H, W);
    FVM_LAUNCH_CHECK();
}

extern "C" int fvm_input_nhwc8_f32(const float* x, void* y, int N, int C, int H, int W, void* stream) {
    return input_nhwc8_launch(x, y, N, C, H, W, stream);
}
extern "C" int fvm_input_nhwc8_f16(const void* x, void* y, int N, int C, int H, int W, void* stream) {
    return input_nhwc8_launch(static_cast<const __half*>(x), y, N, C, H, W, stream);
}
extern "C" int fvm_input_nhwc8_split_f32(const float* x, void* y, int N, int C, int H, int W, void* stream) {
    return input_nhwc8_split_launch(x, y, N, C, H, W, stream);
}
extern "C" int fvm_input_nhwc8_split_f16(const void* x, void* y, int N, int C, int H, int W, void* stream) {
    return input_nhwc8_split_launch(static_cast<const __half*>(x), y, N, C, H, W, stream);
}

// 3x3 window with the loops unrolled: the (up to) nine 16-byte loads of a thread are independent and all in flight
// together; the general kernel above issues them one by one behind its bounds checks. Same mapping, same bits.
__global__ void maxpool3x3_kernel(const __half* __restrict__ x, __half* __restrict__ y, int H, int W, int C, int sh, int sw,
                                  int ph, int pw, int P, int Q, long long total, int rev) {
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    if (rev) i = total - 1 - i;      // last outputs first: see fvm_maxpool_f16
    const int cv = C >> 3;
    const int v = static_cast<int>(i % cv);
    long long t = i / cv;
    const int q = static_cast<int>(t % Q);
    t /= Q;
    const int pp = static_cast<int>(t % P);
    const long long n = t / P;
    const int h0 = pp * sh - ph, w0 = q * sw - pw;
    const uint4 ninf4 = make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);
    V8 a[9];
#pragma unroll
    for (int r = 0; r < 3; ++r) {
#pragma unroll
        for (int s = 0; s < 3; ++s) {
            const int h = h0 + r, w = w0 + s;
            const bool ok = h >= 0 && h < H && w >= 0 && w < W;
            a[r * 3 + s].u = ok ? ldg16(x + ((n * H + h) * W + w) * C + v * 8) : ninf4;
        }
    }
    V8 m;
    m.u = a[0].u;
#pragma unroll
    for (int k = 1; k < 9; ++k) {
#pragma unroll
        for (int j = 0; j < 4; ++j) m.h2[j] = __hmax2(m.h2[j], a[k].h2[j]);
    }
    stg16(y + i * 8, m.u);
}

extern "C" int fvm_maxpool_f16(const void* x, void* y, int N, int H, int W, int C, int kh, int kw, int sh, int sw,
                               int ph, int pw, int P, int Q, void* stream) {
    if (!x || !y || N <= 0 || H <= 0 || W <= 0 || C <= 0 || (C & 7) || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 ||
        P <= 0 || Q <= 0 || !aligned16(x) || !aligned16(y))
        return FVM_ERR_ARG;
    if (kh == 3 && kw == 3) {
        const long long total3 = static_cast<long long>(N) * P * Q * (C >> 3);
        // An input larger than half of the L2 was written front to back by the kernel before: its tail is what the
        // L2 still holds, so the pool walks from the last output to the first (FVM_B200_REVERSE=0: never).
        static const int rev_rule = [] { const char* v = getenv("FVM_B200_REVERSE"); return (v && v[0] == '0') ? 0 : 1; }();
        const int rev = rev_rule && static_cast<long long>(N) * H * W * C * 2 > 64ll * 1024 * 1024;
        maxpool3x3_kernel<<<blocks_for(total3, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const __half*>(x), static_cast<__half*>(y), H, W, C, sh, sw, ph, pw, P, Q, total3, rev);
        FVM_LAUNCH_CHECK();
    }
    const long long total = static_cast<long long>(N) * P * Q * (C >> 3);
    maxpool_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), H, W, C, kh, kw, sh, sw, ph, pw, P, Q, total);
    FVM_LAUNCH_CHECK();
}

extern "C" int fvm_avgpool_f16(const void* x, void* y, int N, int H, int W, int C, int kh, int kw, int sh, int sw,
                               int ph, int pw, int P, int Q, int count_include_pad, void* stream) {
    if (!x || !y || N <= 0 || H <= 0 || W <= 0 || C <= 0 || (C & 7) || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 ||
        P <= 0 || Q <= 0 || !aligned16(x) || !aligned16(y))
        return FVM_ERR_ARG;
    const long long total = static_cast<long long>(N) * P * Q * (C >> 3);
    avgpool_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), H, W, C, kh, kw, sh, sw, ph, pw, P, Q,
        count_include_pad, total);
    FVM_LAUNCH_CHECK();
}

extern "C" long long fvm_gap_scratch_floats(int N, int HW, int C) {
    if (N <= 0 || HW <= 0 || C <= 0) return 0;
    DeviceState* st = device_state();
    const int sms = st ? st->sms : 148;
    return static_cast<long long>(N) * gap_splits(N, HW, C, sms) * C;
}

// Both global-average-pool entry points launch through here; `partial` is the fp32 scratch of stage 1.
static int gap_launch(const void* x, void* y, float* partial, int N, int HW, int C, long long ldx, int splits,
                      void* stream) {
    const int chunk = (HW + splits - 1) / splits;
    const float inv_hw = 1.f / static_cast<float>(HW);
    dim3 grid(((C >> 3) + GAP_VX - 1) / GAP_VX, splits, N), block(GAP_VX, GAP_RY);
    gap_partial_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), partial, HW, C, ldx, splits, chunk, splits == 1 ? static_cast<__half*>(y) : nullptr,
        inv_hw);
    count_launch();
    if (splits > 1) {
        const long long total = static_cast<long long>(N) * C;
        gap_final_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            partial, static_cast<__half*>(y), C, splits, inv_hw, total);
        count_launch();
    }
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}

extern "C" int fvm_global_avgpool_f16(const void* x, void* y, float* partial, int N, int HW, int C, long long ldx,
                                      void* stream) {
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    if (!x || !y || !partial || N <= 0 || HW <= 0 || C <= 0 || (C & 7) || (ldx & 7) || ldx < C || !aligned16(x))
        return FVM_ERR_ARG;
    if (N > 65535) return FVM_ERR_ARG;
    return gap_launch(x, y, partial, N, HW, C, ldx, gap_splits(N, HW, C, st->sms), stream);
}

static int se_gate_launch(const void* g, int slots, const void* w1, const void* b1, const void* w2, const void* b2, void* s,
                          int N, int C, int Cs, int act, float mean_scale, void* stream) {
    if (!g || !w1 || !w2 || !s || N <= 0 || C <= 0 || Cs <= 0 || (C & 7) || (Cs & 7) || act < 0 || act > 6 || slots < 1 ||
        !aligned16(w1) || !aligned16(w2))
        return FVM_ERR_ARG;
    // runs of slots summed in parallel: enough to keep all threads busy, within the static shared-memory limit
    int sgroups = mean_scale != 0.f ? slots / 16 : 0;
    if (mean_scale != 0.f && sgroups < 1) sgroups = 1;
    if (sgroups > 8) sgroups = 8;
    while (sgroups > 1 && static_cast<size_t>(C) * (1 + sgroups) + Cs > 12 * 1024 - 64) --sgroups;
    const size_t smem = (static_cast<size_t>(C) * (1 + sgroups) + Cs) * sizeof(float);
    if (smem > 48 * 1024) return FVM_ERR_ARG;
    DeviceState* st = device_state();
    const int sms = st ? st->sms : 148;
    // large layers: 1024 threads (the loops are latency-bound: more rows / outputs in flight per SM), one block per SM
    const int threads = static_cast<long long>(C) * Cs >= 16 * 1024 ? 1024 : 256;
    const int resident = threads == 1024 ? sms : 2 * sms;
    int split = 1;                       // blocks per image: fill the GPU when the batch alone does not, in one wave
    while (split < 4 && N * split * 2 <= resident && C / (split * 2) >= 256) split *= 2;
    se_gate_kernel<<<dim3(N, split), threads, smem, static_cast<cudaStream_t>(stream)>>>(
        g, static_cast<const __half*>(w1), static_cast<const __half*>(b1), static_cast<const __half*>(w2),
        static_cast<const __half*>(b2), static_cast<__half*>(s), C, Cs, act, mean_scale, slots, sgroups);
    FVM_LAUNCH_CHECK();
}

extern "C" int fvm_se_gate_f16(const void* g, const void* w1, const void* b1, const void* w2, const void* b2, void* s,
                               int N, int C, int Cs, int act, float mean_scale, void* stream) {
    return se_gate_launch(g, 1, w1, b1, w2, b2, s, N, C, Cs, act, mean_scale, stream);
}

extern "C" int fvm_se_gate_pooled_f16(const float* partial, int slots, const void* w1, const void* b1, const void* w2,
                                      const void* b2, void* s, int N, int C, int Cs, int act, float mean_scale,
                                      void* stream) {
    if (mean_scale == 0.f) return FVM_ERR_ARG;
    return se_gate_launch(partial, slots, w1, b1, w2, b2, s, N, C, Cs, act, mean_scale, stream);
}

extern "C" int fvm_gate_weights_f16(const void* w, const void* s, void* out, int N, int K, int C, void* stream) {
    if (!w || !s || !out || N <= 0 || K <= 0 || C <= 0 || (C & 7) || !aligned16(w) || !aligned16(s) || !aligned16(out))
        return FVM_ERR_ARG;
    const long long total = static_cast<long long>(N) * K * (C >> 3);
    gate_weights_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(w), static_cast<const __half*>(s), static_cast<__half*>(out), K, C, total);
    FVM_LAUNCH_CHECK();
}

extern "C" int fvm_se_scale_f16(const void* x, const void* s, void* y, int N, int HW, int C, void* stream) {
    if (!x || !s || !y || N <= 0 || HW <= 0 || C <= 0 || (C & 7) || !aligned16(x) || !aligned16(y) || !aligned16(s))
        return FVM_ERR_ARG;
    const long long total = static_cast<long long>(N) * HW * (C >> 3);
    se_scale_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(s), static_cast<__half*>(y), HW, C, total);
    FVM_LAUNCH_CHECK();
}

template <int G, int VPL>
static void launch_ln(const void* x, const void* gamma, const void* beta, void* y, long long rows, int C, float eps,
                      long long ldx, long long ldy, cudaStream_t stream) {
    constexpr int RPG = VPL >= 3 ? 2 : 4;           // rows in flight per lane group (registers: RPG * VPL * 8 floats)
    constexpr int WARPS = 4;
    const long long rows_per_block = static_cast<long long>(WARPS) * (32 / G) * RPG;
    layernorm_cl_kernel<G, VPL, RPG><<<blocks_for(rows, static_cast<int>(rows_per_block)), WARPS * 32, 0, stream>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(gamma), static_cast<const __half*>(beta),
        static_cast<__half*>(y), rows, C, eps, ldx, ldy);
    count_launch();
}

template <int G>
static bool launch_ln_g(int vpl, const void* x, const void* gamma, const void* beta, void* y, long long rows, int C,
                        float eps, long long ldx, long long ldy, cudaStream_t st) {
    switch (vpl) {
        case 1: launch_ln<G, 1>(x, gamma, beta, y, rows, C, eps, ldx, ldy, st); return true;
        case 2: launch_ln<G, 2>(x, gamma, beta, y, rows, C, eps, ldx, ldy, st); return true;
        case 3: launch_ln<G, 3>(x, gamma, beta, y, rows, C, eps, ldx, ldy, st); return true;
        case 4: launch_ln<G, 4>(x, gamma, beta, y, rows, C, eps, ldx, ldy, st); return true;
    }
    return false;
}

extern "C" int fvm_layernorm_cl_f16(const void* x, const void* gamma, const void* beta, void* y, long long rows, int C,
                                    float eps, long long ldx, long long ldy, void* stream) {
    if (!x || !y || rows <= 0 || C <= 0 || (C & 7) || (ldx & 7) || (ldy & 7) || ldx < C || ldy < C || !aligned16(x) ||
        !aligned16(y) || !aligned16(gamma) || !aligned16(beta))
        return FVM_ERR_ARG;
    const int cv = C >> 3;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // smallest lane group whose lanes hold at most 4 vectors each; rows wider than 128 vectors: 32 lanes x 6 or 8
    bool ok = false;
    if (cv <= 16) ok = launch_ln_g<4>((cv + 3) / 4, x, gamma, beta, y, rows, C, eps, ldx, ldy, st);
    else if (cv <= 32) ok = launch_ln_g<8>((cv + 7) / 8, x, gamma, beta, y, rows, C, eps, ldx, ldy, st);
    else if (cv <= 64) ok = launch_ln_g<16>((cv + 15) / 16, x, gamma, beta, y, rows, C, eps, ldx, ldy, st);
    else if (cv <= 128) ok = launch_ln_g<32>((cv + 31) / 32, x, gamma, beta, y, rows, C, eps, ldx, ldy, st);
    else if (cv <= 192) { launch_ln<32, 6>(x, gamma, beta, y, rows, C, eps, ldx, ldy, st); ok = true; }
    else if (cv <= 256) { launch_ln<32, 8>(x, gamma, beta, y, rows, C, eps, ldx, ldy, st); ok = true; }
    if (!ok) return FVM_ERR_ARG;
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}

extern "C" int fvm_bias_act_f16(void* y, const void* bias, const void* res, long long pixels, int C, int relu,
                                void* stream) {
    if (!y || pixels <= 0 || C <= 0 || (C & 7) || !aligned16(y) || !aligned16(bias) || !aligned16(res))
        return FVM_ERR_ARG;
    const long long total = pixels * (C >> 3);
    bias_act_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half*>(y), static_cast<const __half*>(bias), static_cast<const __half*>(res), C, relu, total);
    FVM_LAUNCH_CHECK();
}

extern "C" int fvm_affine_act_f16(const void* x, const float* scale, const float* shift, void* y, long long pixels,
                                  int C, long long ldx, long long ldy, int act, void* stream) {
    if (!x || !y || !scale || !shift || pixels <= 0 || C <= 0 || (C & 7) || (ldx & 7) || (ldy & 7) || ldx < C ||
        ldy < C || act < 0 || act > 6 || !aligned16(x) || !aligned16(y))
        return FVM_ERR_ARG;
    const long long total = pixels * (C >> 3);
    affine_act_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), scale, shift, static_cast<__half*>(y), C, ldx, ldy, act, total);
    FVM_LAUNCH_CHECK();
}

extern "C" int fvm_add_act_f16(const void* a, const void* b, void* y, long long n, int act, void* stream) {
    if (!a || !b || !y || n <= 0 || (n & 7) || act < 0 || act > 6 || !aligned16(a) || !aligned16(b) || !aligned16(y))
        return FVM_ERR_ARG;
    const long long total = n >> 3;
    add_act_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(a), static_cast<const __half*>(b), static_cast<__half*>(y), act, total);
    FVM_LAUNCH_CHECK();
}

static float resize_scale(int in, int out, int align, float sf) {
    if (align) return out > 1 ? static_cast<float>(in - 1) / static_cast<float>(out - 1) : 0.f;
    if (sf > 0.f) return 1.f / sf;
    return static_cast<float>(in) / static_cast<float>(out);
}

extern "C" int fvm_bilinear_f16(const void* x, const void* base, void* y, int N, int h, int w, int C, int H, int W,
                                int align, float sf_h, float sf_w, int relu, long long ldx, long long ldy,
                                void* stream) {
    if (!x || !y || N <= 0 || h <= 0 || w <= 0 || H <= 0 || W <= 0 || C <= 0 || (C & 7) || (ldx & 7) || (ldy & 7) ||
        ldx < C || ldy < C || !aligned16(x) || !aligned16(y) || !aligned16(base))
        return FVM_ERR_ARG;
    const long long total = static_cast<long long>(N) * H * W * (C >> 3);
    bilinear_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(base), static_cast<__half*>(y), h, w, C, H, W, align,
        resize_scale(h, H, align, sf_h), resize_scale(w, W, align, sf_w), relu, ldx, ldy, total);
    FVM_LAUNCH_CHECK();
}

extern "C" int fvm_up_argmax_f16(const void* s, int32_t* out, int N, int h, int w, int C, long long ld, int H, int W,
                                 int align, void* stream) {
    if (!s || !out || N <= 0 || h <= 0 || w <= 0 || H <= 0 || W <= 0 || C <= 0 || (ld & 7) || ld < C || !aligned16(s))
        return FVM_ERR_ARG;
    if (((C + 7) & ~7) > ld) return FVM_ERR_ARG;   // whole 16-byte vectors are read
    // power-of-two upsample without corner alignment: one thread per group of SF output pixels between two source columns
    static const int use_groups = [] { const char* v = getenv("FVM_B200_UP_GROUPS"); return (v && v[0] == '0') ? 0 : 1; }();
    if (use_groups && !align && w > 0 && H % h == 0 && W % w == 0 && H / h == W / w) {
        const int sf = W / w;
        const long long groups = static_cast<long long>(N) * H * (w + 1);
        const float sch = resize_scale(h, H, 0, 0.f), scw = resize_scale(w, W, 0, 0.f);
        const __half* sp = static_cast<const __half*>(s);
        cudaStream_t st_ = static_cast<cudaStream_t>(stream);
        if (sf == 2) { up_argmax_group_kernel<2><<<blocks_for(groups, 256), 256, 0, st_>>>(sp, out, h, w, C, ld, H, W, sch, scw, groups); FVM_LAUNCH_CHECK(); }
        if (sf == 4) { up_argmax_group_kernel<4><<<blocks_for(groups, 256), 256, 0, st_>>>(sp, out, h, w, C, ld, H, W, sch, scw, groups); FVM_LAUNCH_CHECK(); }
        if (sf == 8) { up_argmax_group_kernel<8><<<blocks_for(groups, 256), 256, 0, st_>>>(sp, out, h, w, C, ld, H, W, sch, scw, groups); FVM_LAUNCH_CHECK(); }
        if (sf == 16) { up_argmax_group_kernel<16><<<blocks_for(groups, 256), 256, 0, st_>>>(sp, out, h, w, C, ld, H, W, sch, scw, groups); FVM_LAUNCH_CHECK(); }
    }
    const long long total = static_cast<long long>(N) * H * W;
    up_argmax_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(s), out, h, w, C, ld, H, W, align, resize_scale(h, H, align, 0.f),
        resize_scale(w, W, align, 0.f), total);
    FVM_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------- allocation-free GAP
// Global average pool for callers that must not allocate: the fp32 partial sums live in a fixed array inside the
// library image instead of a caller-provided scratch buffer. Every GPU that loads the library carries the array
// (FVM_GAP_NOALLOC_MAX_FLOATS * 4 bytes = 4 MiB) until the process exits.
#define FVM_GAP_NOALLOC_MAX_FLOATS (1 << 20)
static __device__ __align__(256) float g_gap_noalloc_scratch[FVM_GAP_NOALLOC_MAX_FLOATS];

namespace {
struct NoAllocGapState {
    float* scratch = nullptr;   // device address of g_gap_noalloc_scratch on this device
    int sms = 0;
    bool ready = false;
};
NoAllocGapState g_noalloc_gap[64];
std::mutex g_noalloc_gap_mutex;
}  // namespace

extern "C" long long fvm_global_avgpool_f16_noalloc_max_floats(void) { return FVM_GAP_NOALLOC_MAX_FLOATS; }

extern "C" int fvm_global_avgpool_f16_noalloc(const void* x, void* y, int N, int HW, int C, long long ldx,
                                              void* stream) {
    if (!x || !y || N <= 0 || N > 65535 || HW <= 0 || C <= 0 || (C & 7) || (ldx & 7) || ldx < C || !aligned16(x))
        return FVM_ERR_ARG;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FVM_ERR_SETUP;
    NoAllocGapState& st = g_noalloc_gap[dev];
    {
        // the first call on a device publishes {scratch, sms, ready} under a lock: two host threads may make it at once
        std::lock_guard<std::mutex> lock(g_noalloc_gap_mutex);
        if (!st.ready) {
            // First call on this device (it is the current device): in host code the array's name is only a handle,
            // the address a kernel can use comes from the runtime. Nothing is allocated here.
            float* ptr = nullptr;
            if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_gap_noalloc_scratch) != cudaSuccess || !ptr)
                return FVM_ERR_SETUP;
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
                return FVM_ERR_SETUP;
            st.scratch = ptr;
            st.sms = sms;
            st.ready = true;
        }
    }
    const int splits = gap_splits(N, HW, C, st.sms);
    if (static_cast<long long>(N) * splits * C > FVM_GAP_NOALLOC_MAX_FLOATS) return FVM_ERR_ARG;   // beyond the fixed scratch
    // stage 1 overwrites every partial sum stage 2 reads: nothing in the shared array has to start at zero
    return gap_launch(x, y, st.scratch, N, HW, C, ldx, splits, stream);
}
