// Dense NHWC fp16 convolution as a persistent, warp-specialised tcgen05 implicit GEMM for sm_100a.
//
//   D[M = N*P*Q, K] = A[M, R*S*C] * W[K, R*S*C]^T      (fp16 operands, fp32 accumulator in TMEM)
//   y = act((D + bias) * scale + res)                  (fp32 epilogue, one rounding to fp16)
//
// Arithmetic contract of the reference op this replaces: classification/fast/csrc/fused_conv.cu:81-99 (epilogue order
// bias -> residual -> activation -> single fp16 rounding); the reference accumulates in fp16 (:50), this kernel in fp32.
//
// Roles: warp 0 = TMA producer (one elected lane), warp 1 = TMEM owner + MMA issuer (one elected lane),
// warps 2..9 = epilogue (TMEM lane group = warp % 4, two warps per group), warp 10 = TMA store issuer (one lane).
//   A tiles: 128 output pixels x 64 input channels per k-block. 1x1 stride-1 convs read them with a 2-D tiled tensor
//            map over [M, C]; every other shape uses an im2col-mode tensor map over the NHWC activation, so padding,
//            stride and dilation are resolved by the TMA unit and out-of-image taps arrive as zeros.
//   B tiles: BN output channels x 64 input channels of one filter tap, 3-D tiled map over [K][R*S][C].
//   Both land in shared memory in the 128-byte-swizzled K-major layout tcgen05.mma consumes directly.
//   Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
//   The residual tile is prefetched by TMA into a swizzled staging buffer, combined in place with the accumulator,
//   and the finished tile leaves by TMA store: the epilogue threads never touch global memory except for the bias.
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
static constexpr int EPI_SPLIT = 2;          // epilogue warps per TMEM lane group (they interleave 32-column chunks)
static constexpr int EPI_WARPS = 4 * EPI_SPLIT;
static constexpr int STORE_WARP = 2 + EPI_WARPS;
static constexpr int CONV_THREADS = 32 * (STORE_WARP + 1);   // producer, MMA, epilogue warps, store warp
static constexpr int MAX_BIAS_BYTES = 16 * 1024;
static constexpr int MAX_STAGES = 8;
static constexpr int MAX_EPI = 3;     // staging buffers for residual-in / output-out tiles
static constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;   // 16 KB
static constexpr uint32_t SUB_BYTES = BM * 64 * 2;       // one 128-row x 64-channel staging sub-tile, 16 KB

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
    int nsub;      // 64-channel staging sub-tiles per output tile = ceil(BN / 64)
    int nepi;      // staging buffers (2 or 3)
    int im2col;    // 0: A via 2-D tiled map over [M, C]; 1: A via im2col map over [N, H, W, C]
    int act;
    int has_res;
    int bias_elems;   // n_tiles * BN: length of the zero-padded bias copy in shared memory
    const __half* bias;
    const float* scale;
    int* status;
};

// status codes written by the device when a bounded wait ran out: 0x100 + role
static constexpr int STATUS_WAIT_PRODUCER = 0x101;
static constexpr int STATUS_WAIT_MMA = 0x102;
static constexpr int STATUS_WAIT_EPILOGUE = 0x103;
static constexpr int STATUS_WAIT_STORE = 0x104;

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
}

// One 8-channel group of one output row: accumulator + bias (+ scale) (+ residual) -> activation -> fp16, combined in
// place with the staged residual chunk at `addr`. ACT: 0 none, 1 relu, 2 = read p.act at run time.
template <int ACT, bool RES, int J>
__device__ __forceinline__ void epilogue_group(const ConvParams& p, const uint32_t (&v)[32], uint32_t addr,
                                               uint32_t bias_addr, int n) {
    float f[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(v[8 * J + k]);
    {
        const uint4 b = lds128(bias_addr);
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 t = unpack_h2(bw[k]);
            f[2 * k] += t.x;
            f[2 * k + 1] += t.y;
        }
    }
    if (p.scale) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.scale + n));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.scale + n + 4));
        f[0] *= s0.x; f[1] *= s0.y; f[2] *= s0.z; f[3] *= s0.w;
        f[4] *= s1.x; f[5] *= s1.y; f[6] *= s1.z; f[7] *= s1.w;
    }
    if (RES) {
        const uint4 r = lds128(addr);
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 t = unpack_h2(rw[k]);
            f[2 * k] += t.x;
            f[2 * k + 1] += t.y;
        }
    }
    if (ACT == 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = fmaxf(f[k], 0.f);
    } else if (ACT == 2) {
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = act_f(f[k], p.act);
    }
    sts128(addr, make_uint4(pack_h2(f[0], f[1]), pack_h2(f[2], f[3]), pack_h2(f[4], f[5]), pack_h2(f[6], f[7])));
}

// The 32-column chunks chunk0, chunk0 + EPI_SPLIT, ... of this thread's row: TMEM -> registers -> staged tile.
template <int ACT, bool RES>
__device__ __forceinline__ void epilogue_rows(const ConvParams& p, uint32_t t_row, uint32_t buf, uint32_t row_xor,
                                              uint32_t bias_base, int n0, int ncols, int chunk0) {
    for (int c0 = chunk0 * 32; c0 < ncols; c0 += 32 * EPI_SPLIT) {
        uint32_t v[32];
        __syncwarp();
        if (c0 + 32 <= p.BN) {
            tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c0), v);
            tmem_ld_wait();
        } else {   // BN is a multiple of 16: the last chunk of a tile may be 16 columns wide
            uint32_t lo[16];
            tmem_ld_32x32b_x16(t_row + static_cast<uint32_t>(c0), lo);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 16; ++k) { v[k] = lo[k]; v[16 + k] = 0u; }
        }
        // 16-byte chunk (col & 63) / 8 of this row inside sub-tile col / 64, 128-byte swizzle
        const uint32_t sub_addr = buf + static_cast<uint32_t>(c0 >> 6) * SUB_BYTES;
        const uint32_t ch0 = static_cast<uint32_t>((c0 & 63) >> 3);
        const uint32_t bias_addr = bias_base + static_cast<uint32_t>(n0 + c0) * 2u;
        const int n = n0 + c0;
        const int left = ncols - c0;   // multiple of 8, > 0
        epilogue_group<ACT, RES, 0>(p, v, sub_addr + (((ch0 + 0) ^ row_xor) << 4), bias_addr, n);
        if (left > 8) epilogue_group<ACT, RES, 1>(p, v, sub_addr + (((ch0 + 1) ^ row_xor) << 4), bias_addr + 16u, n + 8);
        if (left > 16) epilogue_group<ACT, RES, 2>(p, v, sub_addr + (((ch0 + 2) ^ row_xor) << 4), bias_addr + 32u, n + 16);
        if (left > 24) epilogue_group<ACT, RES, 3>(p, v, sub_addr + (((ch0 + 3) ^ row_xor) << 4), bias_addr + 48u, n + 24);
    }
}

// Shared memory map (after rounding the base up to 1024 bytes):
//   [stages x (A tile 16 KB | B tile BN*128 B)] [nepi x nsub x 16 KB staging] [barriers] [tmem slot, abort flag]
//   [bias copy, fp16, zero-padded to n_tiles*BN]
// Staging sub-tiles use the same 128-byte swizzle as the TMA maps of the residual and the output, so the residual
// arrives by TMA load, is combined in place by the epilogue threads (one row each, conflict-free 16-byte accesses)
// and leaves by TMA store: every byte of global traffic of this kernel is a bulk copy.
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_r, const __grid_constant__ CUtensorMap tmap_y,
                    const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_stage_bytes = static_cast<uint32_t>(p.BN) * BK * 2;
    const uint32_t stage_bytes = A_STAGE_BYTES + b_stage_bytes;
    const uint32_t epi_base = smem_base + static_cast<uint32_t>(p.stages) * stage_bytes;
    const uint32_t epi_bytes = static_cast<uint32_t>(p.nsub) * SUB_BYTES;
    const uint32_t bar_base = epi_base + static_cast<uint32_t>(p.nepi) * epi_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + 2 + a); };
    auto res_full_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 4 + e); };
    auto epi_done_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 4 + MAX_EPI + e); };
    auto epi_free_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 4 + 2 * MAX_EPI + e); };
    const uint32_t misc_off = (bar_base - smem_u32(smem_raw)) + 8u * (2 * MAX_STAGES + 4 + 3 * MAX_EPI);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + misc_off + 4);
    // bar_base is 1024-aligned; 29 barriers (232 bytes) + tmem slot + abort flag = 240 bytes: the bias copy that follows
    // is 16-byte aligned, as its 128-bit shared loads require
    static_assert((8 * (2 * MAX_STAGES + 4 + 3 * MAX_EPI) + 8) % 16 == 0, "bias copy must be 16-byte aligned");
    const uint32_t bias_off = misc_off + 8;
    {
        __half* bias_s = reinterpret_cast<__half*>(smem_raw + bias_off);
        for (int i = threadIdx.x; i < p.bias_elems; i += CONV_THREADS)
            bias_s[i] = (p.bias != nullptr && i < p.K) ? p.bias[i] : __float2half_rn(0.f);
    }
    const uint32_t bias_base = smem_u32(smem_raw) + bias_off;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), EPI_WARPS);   // one arrival per epilogue warp
        }
        for (int e = 0; e < p.nepi; ++e) {
            mbar_init(res_full_bar(e), 1);
            mbar_init(epi_done_bar(e), EPI_WARPS);
            mbar_init(epi_free_bar(e), 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_y);
        if (p.has_res) tma_prefetch_desc(&tmap_r);
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
            int e = 0;
            uint32_t e_phase = 0;   // one parity bit per staging buffer
            bool ok = true;
            const int PQ = p.P * p.Q;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int m_tile = tile / p.n_tiles;
                const int n_tile = tile - m_tile * p.n_tiles;
                const int m0 = m_tile * BM;
                const int n0 = n_tile * p.BN;
                if (p.has_res) {
                    // residual tile of this output tile -> staging buffer e (free once its previous store was read out)
                    if (!mbar_wait(epi_free_bar(e), ((e_phase >> e) & 1u) ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    e_phase ^= 1u << e;
                    const int nsub = min(p.nsub, (p.K - n0 + 63) >> 6);
                    mbar_expect_tx(res_full_bar(e), static_cast<uint32_t>(nsub) * SUB_BYTES);
                    for (int sub = 0; sub < nsub; ++sub)
                        tma_load_2d(epi_base + static_cast<uint32_t>(e) * epi_bytes + static_cast<uint32_t>(sub) * SUB_BYTES,
                                    &tmap_r, res_full_bar(e), n0 + sub * 64, m0);
                    if (++e == p.nepi) e = 0;
                }
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
            // load of this CTA is still in flight when the CTA exits. (Residual loads are consumed by the epilogue,
            // which the final barrier below waits for.)
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
            uint32_t acc_phase = 0;   // one parity bit per accumulator buffer
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                if (!mbar_wait(tempty_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag)) {
                    atomicExch(p.status, STATUS_WAIT_MMA);
                    ok = false;
                    break;
                }
                acc_phase ^= 1u << acc;
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
    } else if (warp < STORE_WARP) {
        // ------------------------------------------------------------------ epilogue
        // EPI_SPLIT warps share one TMEM lane group (32 rows) and interleave its 32-column chunks.
        const int lane_group = warp & 3;
        const int chunk0 = (warp - 2) >> 2;           // first 32-column chunk of this warp
        const int row = lane_group * 32 + lane;       // row of the tile = TMEM lane
        const uint32_t row_off = static_cast<uint32_t>(row) * 128u;
        const uint32_t row_xor = static_cast<uint32_t>(row & 7);
        uint32_t acc_phase = 0;   // one parity bit per accumulator buffer
        uint32_t e_phase = 0;     // one parity bit per staging buffer
        int e = 0;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const int m_tile = tile / p.n_tiles;
            const int n_tile = tile - m_tile * p.n_tiles;
            const int n0 = n_tile * p.BN;
            // staging buffer: with a residual it is filled by TMA (res_full); without, wait until it is free
            const bool got_buf = p.has_res ? mbar_wait(res_full_bar(e), (e_phase >> e) & 1u, abort_flag)
                                           : mbar_wait(epi_free_bar(e), ((e_phase >> e) & 1u) ^ 1u, abort_flag);
            if (!got_buf || !mbar_wait(tfull_bar(acc), (acc_phase >> acc) & 1u, abort_flag)) {
                if (lane == 0) atomicExch(p.status, STATUS_WAIT_EPILOGUE);
                ok = false;
                break;
            }
            e_phase ^= 1u << e;
            acc_phase ^= 1u << acc;
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                                   static_cast<uint32_t>(acc * p.acc_stride);
            const uint32_t buf = epi_base + static_cast<uint32_t>(e) * epi_bytes + row_off;
            const int ncols = min(p.BN, p.K - n0);   // multiple of 8
            switch ((p.act == 0 ? 0 : (p.act == 1 ? 1 : 2)) * 2 + (p.has_res ? 1 : 0)) {
                case 0: epilogue_rows<0, false>(p, t_row, buf, row_xor, bias_base, n0, ncols, chunk0); break;
                case 1: epilogue_rows<0, true>(p, t_row, buf, row_xor, bias_base, n0, ncols, chunk0); break;
                case 2: epilogue_rows<1, false>(p, t_row, buf, row_xor, bias_base, n0, ncols, chunk0); break;
                case 3: epilogue_rows<1, true>(p, t_row, buf, row_xor, bias_base, n0, ncols, chunk0); break;
                case 4: epilogue_rows<2, false>(p, t_row, buf, row_xor, bias_base, n0, ncols, chunk0); break;
                default: epilogue_rows<2, true>(p, t_row, buf, row_xor, bias_base, n0, ncols, chunk0); break;
            }
            // all TMEM reads of this warp are done: hand the accumulator back; publish this warp's part of the staged
            // tile to the async proxy, then tell the store warp
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(tempty_bar(acc));
                mbar_arrive(epi_done_bar(e));
            }
            if (++e == p.nepi) e = 0;
        }
    } else {
        // ------------------------------------------------------------------ store warp
        if (lane == 0) {
            uint32_t e_phase = 0;   // one parity bit per staging buffer
            int e = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int m_tile = tile / p.n_tiles;
                const int n_tile = tile - m_tile * p.n_tiles;
                const int m0 = m_tile * BM;
                const int n0 = n_tile * p.BN;
                if (!mbar_wait(epi_done_bar(e), (e_phase >> e) & 1u, abort_flag)) {
                    atomicExch(p.status, STATUS_WAIT_STORE);
                    ok = false;
                    break;
                }
                e_phase ^= 1u << e;
                const int nsub = min(p.nsub, (p.K - n0 + 63) >> 6);
                for (int sub = 0; sub < nsub; ++sub)
                    tma_store_2d(&tmap_y, epi_base + static_cast<uint32_t>(e) * epi_bytes + static_cast<uint32_t>(sub) * SUB_BYTES,
                                 n0 + sub * 64, m0);
                tma_store_commit();
                tma_store_wait_read();          // the staging buffer has been read out: it may be refilled
                mbar_arrive(epi_free_bar(e));
                if (++e == p.nepi) e = 0;
            }
            tma_store_wait_all();               // all output bytes are written before the CTA exits
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

// Shared-memory plan for an output-channel tile of BN: staging buffers for the residual/output tiles first (3 if the
// main loop still gets enough stages, else 2), then the zero-padded bias copy, the rest goes to the A/B pipeline.
struct SmemPlan {
    int stages, nepi;
    size_t bytes;
};
static bool plan_smem(int BN, int kblocks, int K, SmemPlan* out) {
    const int n_tiles = (K + BN - 1) / BN;
    const uint32_t stage_bytes = A_STAGE_BYTES + static_cast<uint32_t>(BN) * BK * 2;
    const uint32_t epi_bytes = static_cast<uint32_t>((BN + 63) / 64) * SUB_BYTES;
    const uint32_t bias_bytes = (static_cast<uint32_t>(n_tiles * BN) * 2 + 15u) & ~15u;
    if (bias_bytes > MAX_BIAS_BYTES) return false;
    const uint32_t fixed = 1024 + 8 * (2 * MAX_STAGES + 4 + 3 * MAX_EPI) + 8 + bias_bytes;
    const uint32_t total = 227 * 1024;
    if (fixed + 2 * epi_bytes + 2 * stage_bytes > total) return false;
    const uint32_t budget = total - fixed;
    const int want_stages = kblocks + 1 < 4 ? kblocks + 1 : 4;
    const int nepi = (3 * epi_bytes + static_cast<uint32_t>(want_stages) * stage_bytes <= budget) ? 3 : 2;
    int stages = static_cast<int>((budget - static_cast<uint32_t>(nepi) * epi_bytes) / stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > kblocks + 1) stages = kblocks + 1;   // never more stages than could be in flight
    if (stages < 2) stages = 2;
    out->stages = stages;
    out->nepi = nepi;
    out->bytes = fixed + static_cast<size_t>(stages) * stage_bytes + static_cast<size_t>(nepi) * epi_bytes;
    return true;
}

// Picks the output-channel tile. A single tile over all of K (any multiple of 16 up to 256) reads A once; when K is
// split, tiles must be multiples of 64 channels because the output leaves in 64-channel TMA boxes. Among the
// candidates that fit shared memory the best (wave efficiency x useful-column fraction) wins, larger tiles first;
// a deep reduction (many k-blocks) additionally wants at least 3 pipeline stages.
static int pick_bn(int m_tiles, int K, int kblocks, int sms) {
    const int Kp = (K + 15) / 16 * 16;
    int cands[5];
    int nc = 0;
    if (Kp <= 256) cands[nc++] = Kp;
    const int fixed[3] = {256, 128, 64};
    for (int i = 0; i < 3; ++i)
        if (fixed[i] < Kp) cands[nc++] = fixed[i];
    int best = 0;
    double best_score = -1.0;
    for (int i = 0; i < nc; ++i) {
        const int bn = cands[i];
        SmemPlan sp;
        if (!plan_smem(bn, kblocks, K, &sp)) continue;
        const int nt = (K + bn - 1) / bn;
        const long long tiles = static_cast<long long>(m_tiles) * nt;
        const long long waves = (tiles + sms - 1) / sms;
        const double wave_eff = static_cast<double>(tiles) / static_cast<double>(waves * sms);
        const double col_eff = static_cast<double>(K) / static_cast<double>(nt * bn);
        double score = wave_eff * col_eff;
        if (kblocks >= 8 && sp.stages < 3) score *= 0.8;
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
    p.BN = force_bn > 0 ? force_bn : pick_bn(p.m_tiles, K, p.kblocks, st->sms);
    if (p.BN < 16 || p.BN > 256 || (p.BN & 15)) return FVM_ERR_ARG;
    p.n_tiles = (K + p.BN - 1) / p.BN;
    if (p.n_tiles > 1 && (p.BN & 63)) return FVM_ERR_ARG;   // split K only in whole 64-channel store boxes
    int cols = 32;
    while (cols < 2 * p.BN) cols <<= 1;
    p.tmem_cols = cols;
    p.acc_stride = cols / 2;
    p.im2col = !(R == 1 && S == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0);
    p.act = act;
    p.has_res = res != nullptr;
    p.bias = static_cast<const __half*>(bias);
    p.scale = scale;
    p.status = st->status_dev;
    p.nsub = (p.BN + 63) / 64;

    SmemPlan sp;
    if (!plan_smem(p.BN, p.kblocks, K, &sp)) return FVM_ERR_ARG;
    p.bias_elems = p.n_tiles * p.BN;
    p.stages = sp.stages;
    p.nepi = sp.nepi;
    // Always request more than half of an SM's shared memory: at most one CTA per SM, so the TMEM request of a CTA
    // never waits on a co-resident CTA of the same kernel.
    size_t smem = sp.bytes;
    if (smem < 120 * 1024) smem = 120 * 1024;

    CUtensorMap tmap_a, tmap_b, tmap_r, tmap_y;
    {
        // output [M, K] (row stride ldy) and residual [M, K] (row stride ldr): 64-channel x 128-row boxes
        cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(p.M)};
        cuuint32_t box[2] = {64, BM};
        cuuint32_t estr[2] = {1, 1};
        cuuint64_t ystr[1] = {static_cast<cuuint64_t>(ldy) * 2};
        CUresult r = g_encode_tiled(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, y, dims, ystr, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
        if (res) {
            cuuint64_t rstr[1] = {static_cast<cuuint64_t>(ldr) * 2};
            r = g_encode_tiled(&tmap_r, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(res), dims, rstr, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
        } else {
            tmap_r = tmap_y;
        }
    }
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
    conv_tcgen05_kernel<<<grid, CONV_THREADS, smem, stream>>>(tmap_a, tmap_b, tmap_r, tmap_y, p);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}

}  // namespace fvm
