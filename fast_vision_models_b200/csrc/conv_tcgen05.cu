// Dense NHWC fp16 convolution as a persistent, warp-specialised tcgen05 implicit GEMM for sm_100a.
//
//   D[M = N*P*Q, K] = A[M, R*S*C] * W[K, R*S*C]^T      (fp16 operands, fp32 accumulator in TMEM)
//   y = act((D + bias) * scale + res)                  (fp32 epilogue, one rounding to fp16)
//
// Arithmetic contract of the reference op this replaces: classification/fast/csrc/fused_conv.cu:81-99 (epilogue order
// bias -> residual -> activation -> single fp16 rounding); the reference accumulates in fp16 (:50), this kernel in fp32.
//
// Roles (192 threads): warp 0 = TMA producer (one elected lane), warp 1 = TMEM owner + MMA issuer (one elected lane),
// warps 2..5 = epilogue (TMEM lane group = warp % 4).
//   A tiles: 128 output pixels x 64 input channels per k-block. 1x1 stride-1 convs read them with a 2-D tiled tensor
//            map over [M, C]; every other shape uses an im2col-mode tensor map over the NHWC activation, so padding,
//            stride and dilation are resolved by the TMA unit and out-of-image taps arrive as zeros.
//   B tiles: BN output channels x 64 input channels of one filter tap, 3-D tiled map over [K][R*S][C].
//   Both land in shared memory in the 128-byte-swizzled K-major layout tcgen05.mma consumes directly.
//   Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
// No cluster launch and no multicast: every CTA issues its own loads.
#include <cuda.h>

#include <atomic>
#include <cstdio>
#include <cstring>

#include "fvm_internal.h"
#include "ptx_sm100.cuh"

namespace fvm {

static constexpr int BM = 128;        // output pixels per tile (= TMEM lanes)
static constexpr int BK = 64;         // input channels per k-block (128 bytes of fp16 = one swizzle row)
static constexpr int CONV_THREADS = 192;
static constexpr int MAX_STAGES = 8;
static constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;  // 16 KB

struct ConvParams {
    int M, K, C;
    int R, S, P, Q;
    int sh, sw, ph, pw, dh, dw;
    int cchunks;   // ceil(C / 64)
    int kblocks;   // R * S * cchunks
    int BN;        // output channels per tile (multiple of 16, <= 256)
    int acc_stride;  // TMEM columns between the two accumulator buffers
    int tmem_cols;   // allocated TMEM columns (power of two >= 32)
    int n_tiles, m_tiles, stages;
    int im2col;    // 0: A via 2-D tiled map over [M, C]; 1: A via im2col map over [N, H, W, C]
    int act;
    const __half* bias;
    const __half* res;
    const float* scale;
    __half* y;
    long long ldy, ldr;
    int* status;
};

// status codes written by the device: 0x100 + role (1 producer, 2 mma, 3 epilogue) when a bounded wait ran out
static constexpr int STATUS_WAIT_PRODUCER = 0x101;
static constexpr int STATUS_WAIT_MMA = 0x102;
static constexpr int STATUS_WAIT_EPILOGUE = 0x103;

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
}

__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows (1024 bytes)
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_stage_bytes = static_cast<uint32_t>(p.BN) * BK * 2;
    const uint32_t stage_bytes = A_STAGE_BYTES + b_stage_bytes;
    const uint32_t bar_base = smem_base + static_cast<uint32_t>(p.stages) * stage_bytes;
    // barrier block: full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2], then tmem slot + abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + 2 + a); };
    const uint32_t misc_off = (bar_base - smem_u32(smem_raw)) + 8u * (2 * MAX_STAGES + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + misc_off + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), static_cast<uint32_t>(p.tmem_cols));
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = p.m_tiles * p.n_tiles;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int PQ = p.P * p.Q;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int m_tile = tile / p.n_tiles;
                const int n_tile = tile - m_tile * p.n_tiles;
                const int m0 = m_tile * BM;
                const int n0 = n_tile * p.BN;
                int img = 0, h0 = 0, w0 = 0;
                if (p.im2col) {
                    img = m0 / PQ;
                    const int rem = m0 - img * PQ;
                    const int pp = rem / p.Q;
                    const int qq = rem - pp * p.Q;
                    h0 = pp * p.sh - p.ph;
                    w0 = qq * p.sw - p.pw;
                }
                int tap = 0, cc = 0, r = 0, s = 0;
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + static_cast<uint32_t>(stage) * stage_bytes;
                    const uint32_t b_dst = a_dst + A_STAGE_BYTES;
                    mbar_expect_tx(full_bar(stage), stage_bytes);
                    if (p.im2col) {
                        tma_load_im2col_4d(a_dst, &tmap_a, full_bar(stage), cc * BK, w0, h0, img,
                                           static_cast<uint16_t>(s * p.dw), static_cast<uint16_t>(r * p.dh));
                    } else {
                        tma_load_2d(a_dst, &tmap_a, full_bar(stage), cc * BK, m0);
                    }
                    tma_load_3d(b_dst, &tmap_b, full_bar(stage), cc * BK, tap, n0);
                    if (++cc == p.cchunks) {
                        cc = 0;
                        ++tap;
                        if (++s == p.S) { s = 0; ++r; }
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            // Drain: wait (bounded) until the MMA warp has released every stage this thread filled, so that no bulk
            // copy of this CTA is still in flight when the CTA exits.
            if (ok) {
                for (int i = 0; i < p.stages; ++i) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) break;
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16_f32(BM, p.BN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase[2] = {0, 0};
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag)) {
                    atomicExch(p.status, STATUS_WAIT_MMA);
                    ok = false;
                    break;
                }
                acc_phase[acc] ^= 1u;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.acc_stride);
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_MMA);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_src = smem_base + static_cast<uint32_t>(stage) * stage_bytes;
                    const uint64_t a_desc = umma_desc_sw128(a_src);
                    const uint64_t b_desc = umma_desc_sw128(a_src + A_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // advancing 16 halves (32 bytes) along K inside the swizzle row: +2 in the >>4 address field
                        umma_f16(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k),
                                 idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));   // frees the stage once these MMAs have read it
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(tfull_bar(acc));  // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps = 128 TMEM lanes)
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        uint32_t acc_phase[2] = {0, 0};
        int it = 0;
        bool ok = true;
        const bool vec16 = ((p.ldy & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 31) == 0) &&
                           (p.res == nullptr ||
                            (((p.ldr & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.res) & 31) == 0)));
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const int m_tile = tile / p.n_tiles;
            const int n_tile = tile - m_tile * p.n_tiles;
            const long long m = static_cast<long long>(m_tile) * BM + row_in_tile;
            const int n0 = n_tile * p.BN;
            if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag)) {
                if (lane == 0) atomicExch(p.status, STATUS_WAIT_EPILOGUE);
                ok = false;
                break;
            }
            acc_phase[acc] ^= 1u;
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                                   static_cast<uint32_t>(acc * p.acc_stride);
            const bool row_ok = m < p.M;
            __half* yrow = p.y + m * p.ldy;
            const __half* rrow = p.res ? p.res + m * p.ldr : nullptr;
            const int ncols = min(p.BN, p.K - n0);   // multiple of 8
            for (int c0 = 0; c0 < ncols; c0 += 16) {
                uint32_t v[16];
                __syncwarp();
                tmem_ld_32x32b_x16(t_row + static_cast<uint32_t>(c0), v);   // warp-collective: no divergence here
                tmem_ld_wait();
                if (c0 + 16 >= ncols) {
                    // last TMEM read of this tile: hand the accumulator back before the arithmetic and the stores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(acc));
                }
                if (!row_ok) continue;
                const int n = n0 + c0;
                const int valid = min(16, ncols - c0);   // 8 or 16
                float f[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
                if (p.bias) {
                    const uint4* bp = reinterpret_cast<const uint4*>(p.bias + n);
                    uint4 b0 = __ldg(bp);
                    uint4 b1 = valid > 8 ? __ldg(bp + 1) : make_uint4(0, 0, 0, 0);
                    const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float2 t = unpack_h2(bw[j]);
                        f[2 * j] += t.x;
                        f[2 * j + 1] += t.y;
                    }
                }
                if (p.scale) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (j < valid) f[j] *= __ldg(p.scale + n + j);
                }
                if (rrow) {
                    uint32_t rw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    if (vec16 && valid == 16) {
                        ldg_nc_v8(rrow + n, rw);
                    } else {
                        uint4 r0 = __ldg(reinterpret_cast<const uint4*>(rrow + n));
                        rw[0] = r0.x; rw[1] = r0.y; rw[2] = r0.z; rw[3] = r0.w;
                        if (valid > 8) {
                            uint4 r1 = __ldg(reinterpret_cast<const uint4*>(rrow + n + 8));
                            rw[4] = r1.x; rw[5] = r1.y; rw[6] = r1.z; rw[7] = r1.w;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float2 t = unpack_h2(rw[j]);
                        f[2 * j] += t.x;
                        f[2 * j + 1] += t.y;
                    }
                }
                if (p.act) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) f[j] = act_f(f[j], p.act);
                }
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = pack_h2(f[2 * j], f[2 * j + 1]);
                if (vec16 && valid == 16) {
                    stg_v8(yrow + n, o);
                } else {
                    *reinterpret_cast<uint4*>(yrow + n) = make_uint4(o[0], o[1], o[2], o[3]);
                    if (valid > 8) *reinterpret_cast<uint4*>(yrow + n + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
    }
}

// ---------------------------------------------------------------------------------------------------- host side

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*PFN_encodeIm2col)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                     const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled g_encode_tiled = nullptr;
static PFN_encodeIm2col g_encode_im2col = nullptr;
static int g_driver_version = 0;

// The driver API is reached through the runtime's entry-point query, so the library has no link-time dependency on
// libcuda and still loads on a machine without a driver (where only symbol checks run).
int conv_host_init() {
    if (g_encode_tiled && g_encode_im2col) return FVM_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
        return FVM_ERR_SETUP;
    g_encode_tiled = reinterpret_cast<PFN_encodeTiled>(fn);
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
        return FVM_ERR_SETUP;
    g_encode_im2col = reinterpret_cast<PFN_encodeIm2col>(fn);
    cudaDriverGetVersion(&g_driver_version);
    if (cudaFuncSetAttribute(conv_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
        cudaSuccess)
        return FVM_ERR_SETUP;
    return FVM_OK;
}

// Picks the output-channel tile: the candidate with the best (wave efficiency x useful-column fraction), larger first.
static int pick_bn(int m_tiles, int K, int sms) {
    const int Kp = (K + 15) / 16 * 16;
    int cands[6];
    int nc = 0;
    if (Kp <= 256) cands[nc++] = Kp;
    const int fixed[4] = {256, 128, 64, 32};
    for (int i = 0; i < 4; ++i)
        if (fixed[i] < Kp) cands[nc++] = fixed[i];
    int best = cands[0];
    double best_score = -1.0;
    for (int i = 0; i < nc; ++i) {
        const int bn = cands[i];
        const int nt = (K + bn - 1) / bn;
        const long long tiles = static_cast<long long>(m_tiles) * nt;
        const long long waves = (tiles + sms - 1) / sms;
        const double wave_eff = static_cast<double>(tiles) / static_cast<double>(waves * sms);
        const double col_eff = static_cast<double>(K) / static_cast<double>(nt * bn);
        const double score = wave_eff * col_eff;
        if (score > best_score * 1.05) {   // prefer the larger tile unless a smaller one is clearly better
            best_score = score;
            best = bn;
        }
    }
    return best;
}

int conv2d_launch(const void* x, const void* w, const void* bias, const void* res, const float* scale, void* y, int N,
                  int H, int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                  long long ldx, long long ldy, long long ldr, int act, int force_bn, cudaStream_t stream) {
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    if (!x || !w || !y) return FVM_ERR_ARG;
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || R <= 0 || S <= 0) return FVM_ERR_ARG;
    if ((C & 7) || (K & 7) || (ldx & 7) || (ldy & 7) || (res && (ldr & 7))) return FVM_ERR_ARG;
    if (sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || ph < 0 || pw < 0) return FVM_ERR_ARG;
    if (ldx < C || ldy < K || (res && ldr < K)) return FVM_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(res) & 15) ||
        (reinterpret_cast<uintptr_t>(bias) & 15))
        return FVM_ERR_ARG;
    if (act < 0 || act > 6) return FVM_ERR_ARG;
    const int P = (H + 2 * ph - dh * (R - 1) - 1) / sh + 1;
    const int Q = (W + 2 * pw - dw * (S - 1) - 1) / sw + 1;
    if (P <= 0 || Q <= 0) return FVM_ERR_ARG;
    const long long M_ll = static_cast<long long>(N) * P * Q;
    if (M_ll > 0x7fffff00ll) return FVM_ERR_ARG;

    ConvParams p;
    memset(&p, 0, sizeof(p));
    p.M = static_cast<int>(M_ll);
    p.K = K; p.C = C; p.R = R; p.S = S; p.P = P; p.Q = Q;
    p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
    p.cchunks = (C + BK - 1) / BK;
    p.kblocks = R * S * p.cchunks;
    p.m_tiles = (p.M + BM - 1) / BM;
    p.BN = force_bn > 0 ? force_bn : pick_bn(p.m_tiles, K, st->sms);
    if (p.BN < 16 || p.BN > 256 || (p.BN & 15)) return FVM_ERR_ARG;
    p.n_tiles = (K + p.BN - 1) / p.BN;
    int cols = 32;
    while (cols < 2 * p.BN) cols <<= 1;
    p.tmem_cols = cols;
    p.acc_stride = cols / 2;
    p.im2col = !(R == 1 && S == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0);
    p.act = act;
    p.bias = static_cast<const __half*>(bias);
    p.res = static_cast<const __half*>(res);
    p.scale = scale;
    p.y = static_cast<__half*>(y);
    p.ldy = ldy; p.ldr = ldr;
    p.status = st->status_dev;

    const uint32_t stage_bytes = A_STAGE_BYTES + static_cast<uint32_t>(p.BN) * BK * 2;
    const uint32_t budget = 200 * 1024;
    int stages = static_cast<int>(budget / stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > p.kblocks + 1) stages = p.kblocks + 1;   // never more stages than could be in flight
    if (stages < 2) stages = 2;
    p.stages = stages;
    // Always request more than half of an SM's shared memory: at most one CTA per SM, so the TMEM request of a CTA
    // never waits on a co-resident CTA of the same kernel.
    size_t smem = 1024 + static_cast<size_t>(stages) * stage_bytes + 8 * (2 * MAX_STAGES + 4) + 16;
    if (smem < 120 * 1024) smem = 120 * 1024;

    CUtensorMap tmap_a, tmap_b;
    {
        // weights [K][R*S][C]
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(R * S), static_cast<cuuint64_t>(K)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(C) * 2, static_cast<cuuint64_t>(R) * S * C * 2};
        cuuint32_t box[3] = {BK, 1, static_cast<cuuint32_t>(p.BN)};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = g_encode_tiled(&tmap_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w), dims, strides,
                                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
    }
    if (!p.im2col) {
        cuuint64_t dims[2] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(p.M)};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldx) * 2};
        cuuint32_t box[2] = {BK, BM};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = g_encode_tiled(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides,
                                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
    } else {
        // NHWC activation as (C, W, H, N); the filter-window origin moves inside the box
        // [-pad, size + pad - dilation*(taps-1) - 1], stepping by the conv stride; each load adds the tap offset.
        const int up_w = pw - (S - 1) * dw, up_h = ph - (R - 1) * dh;
        if (pw > 128 || ph > 128 || up_w < -128 || up_h < -128 || (S - 1) * dw > 255 || (R - 1) * dh > 255)
            return FVM_ERR_ARG;
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(N)};
        cuuint64_t strides[3] = {static_cast<cuuint64_t>(ldx) * 2, static_cast<cuuint64_t>(W) * ldx * 2,
                                 static_cast<cuuint64_t>(H) * W * ldx * 2};
        int lower[2] = {-pw, -ph};
        int upper[2] = {up_w, up_h};
        cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(sw), static_cast<cuuint32_t>(sh), 1};
        CUresult r = g_encode_im2col(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(x), dims, strides,
                                     lower, upper, BK, BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
        // Driver releases up to CUDA 13.1 mis-handle im2col maps over tensors smaller than 128 KiB unless bit 21 of
        // the descriptor's second word is cleared (the same correction CUTLASS applies when it builds these maps).
        const unsigned long long bytes = static_cast<unsigned long long>(N) * H * W * ldx * 2;
        if (g_driver_version <= 13010 && bytes < 131072ull)
            reinterpret_cast<uint64_t*>(&tmap_a)[1] &= ~(1ull << 21);
    }

    const long long total_tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
    const int grid = static_cast<int>(total_tiles < st->sms ? total_tiles : st->sms);
    conv_tcgen05_kernel<<<grid, CONV_THREADS, smem, stream>>>(tmap_a, tmap_b, p);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}

}  // namespace fvm
