// Dense NHWC fp16 convolution as a persistent, warp-specialised tcgen05 implicit GEMM for sm_100a.
//
//   D[M = N*P*Q, K] = A[M, R*S*C] * W[K, R*S*C]^T      (fp16 operands, fp32 accumulator in TMEM)
//   y = act((D + bias) * scale + res)                  (fp32 epilogue, one rounding to fp16)
//
// Arithmetic contract of the reference op this replaces: classification/fast/csrc/fused_conv.cu:81-99 (epilogue order
// bias -> residual -> activation -> single fp16 rounding); the reference accumulates in fp16 (:50), this kernel in fp32.
//
// Roles (19 warps): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..17 = four epilogue groups of 4
// warps (TMEM lane group = warp % 4) that share every tile by column chunks, warp 18 = TMA store issuer. The three single-thread
// roles run in one lane chosen by elect.sync, with control flow that depends on kernel parameters only: the compiler
// then keeps their counters and descriptors in uniform registers, which is what tcgen05.mma / TMA instructions read
// (measured: about 50 cycles per issued MMA against about 120 under `if (lane == 0)`).
//   A tiles: 128 output pixels x 64 input channels per k-block. 1x1 stride-1 convs read them with a 2-D tiled tensor
//            map over [M, C]; every other shape uses an im2col-mode tensor map over the NHWC activation, so padding,
//            stride and dilation are resolved by the TMA unit and out-of-image taps arrive as zeros.
//   B tiles: BN output channels x 64 input channels of one filter tap, 3-D tiled map over [K][R*S][C].
//   Both land in shared memory in the 128-byte-swizzled K-major layout tcgen05.mma consumes directly.
//   Two to four accumulator buffers in TMEM let the epilogue of a tile overlap the main loop of the next ones.
//   The residual tile is prefetched by TMA into a swizzled staging buffer, combined in place with the accumulator,
//   and the finished tile leaves by TMA store: the epilogue threads never touch global memory except for the bias.
//   Halo mode (3x3, stride 1): a tile is a 16 x 8 patch of output pixels; its input patch with border is staged once
//   per 64 channels and the nine taps are MMA operands that start at different rows of that patch.
//   Stem mode (stride 2, 8-channel input stored as two column-parity planes per image row): the same idea without
//   swizzle; one MMA covers two vertically adjacent taps.
// conv_tcgen05_kernel and conv_streamk_kernel launch no clusters; in every kernel each CTA issues its own loads.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "fvm_internal.h"
#include "ptx_sm100.cuh"

namespace fvm {

static constexpr int BM = 128;        // output pixels per tile (= TMEM lanes)
static constexpr int BK = 64;         // input channels per k-block (128 bytes of fp16 = one swizzle row)
static constexpr int EPI_GROUPS = 4;         // epilogue groups of 4 warps; group g finishes the 32-column chunks g, g+4, .. of every tile
static constexpr int MAX_ACC = 4;            // TMEM accumulator buffers (4 when a tile is at most 128 columns wide, else 2)
static constexpr int EPI_WARPS = 4 * EPI_GROUPS;
static constexpr int STORE_WARP = 2 + EPI_WARPS;
static constexpr int CONV_THREADS = 32 * (STORE_WARP + 1);   // producer, MMA, epilogue warps, store warp
static constexpr int MAX_BIAS_BYTES = 16 * 1024;
static constexpr int EPI_BACKOFF_NS = 64;     // sleep between polls of the epilogue / store warps
static constexpr int MAX_STAGES = 8;
static constexpr int MAX_EPI = 6;     // staging buffers for residual-in / output-out tiles
static constexpr int MAX_HALO = 3;    // halo-tile buffers (3x3 stride-1 mode)
static constexpr int NUM_BARRIERS = 2 * MAX_STAGES + 2 * MAX_ACC + 3 * MAX_EPI + 1 + 2 * MAX_HALO;   // stages, accumulators, staging, resident B, halo
static constexpr int HALO_TH = 16, HALO_TW = 8;   // output patch of a halo-mode tile: 16 rows x 8 columns = 128 pixels
static constexpr int HALO_PITCH = 16;             // pixels per staged halo row (a multiple of 8: 8-row groups stay 1024-aligned)
static constexpr int MISC_BYTES = 16 + (NUM_BARRIERS & 1) * 8;   // tmem slot, abort flag; keeps what follows 16-byte aligned
static constexpr int TAPS_PER_KBLOCK = 8;                    // tap-packed mode, 8-channel taps: 8 taps x 8 channels = 64 K elements
static constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;   // 16 KB
static constexpr uint32_t SUB_BYTES = BM * 64 * 2;       // one 128-row x 64-channel staging sub-tile, 16 KB

struct ConvParams {
    int M, K, C;
    int R, S, P, Q;
    int sh, sw, ph, pw, dh, dw;
    int cchunks;   // ceil(C / 64)
    int kblocks;   // R * S * cchunks
    int BN;        // output channels per tile (multiple of 32, <= 256)
    int acc_stride;  // TMEM columns between accumulator buffers
    int nacc;        // accumulator buffers in TMEM (2 or 4)
    int tmem_cols;   // allocated TMEM columns (power of two >= 32)
    int n_tiles, m_tiles, stages;
    int mt;        // 128-row sub-tiles per (macro) tile: 1, 2 or 4; a tile is 128*mt output pixels x BN channels
    int a_loads, a_rows;   // tiled-mode A loads per k-block and rows per load (a TMA box has at most 256 rows)
    int nsub;      // 64-channel staging sub-tiles per 128-row sub-tile = ceil(BN / 64)
    int nepi;      // staging buffers (1..6)
    int im2col;    // 0: A via 2-D tiled map over [M, C]; 1: A via im2col map over [N, H, W, C]
    int tapk;      // 8 or 16: "tap-packed" mode for inputs of 8 / 16 channels: a k-block is 8 / 4 filter taps of that
                   // many channels (64 K elements), weights resident in smem; 0: one tap of 64 channels per k-block
    int taps;      // R * S
    int halo;      // 1: 3x3 stride-1 'halo' mode: a tile is a 16x8 pixel patch of one image; its input patch (+ border) is
                   // staged once per 64 channels and the 9 taps are shifted views of it (9x fewer L2 reads than im2col)
                   // 2: stride-2 stem over an 8-channel input stored as two column-parity planes per image row: the
                   // input patch of a 16x8 output patch is staged once, every filter tap is a shifted view of it
    int halo_rows, nh, tiles_x, tiles_y;   // staged rows (16 + 2*dilation), halo buffers, patches per image row / column
    uint32_t hbytes, htx;                  // staged-patch buffer stride / bytes per load
    int stem_taps, stem_xlo;               // stem mode: weight taps held (R rounded up to even, times S); leftmost plane column
    uint32_t stem_prow;                    // stem mode: bytes per staged input row (two planes)
    FastDiv div_txy, div_tx;
    int bres;      // 1: the weights of this CTA's n-tile stay resident in shared memory (loaded once); each CTA keeps one
                   // n-tile and walks the m-tiles; pipeline stages then hold A only
    int act;
    int has_res;
    int bias_elems;   // n_tiles * BN: length of the zero-padded bias copy in shared memory
    FastDiv div_ntiles, div_pq, div_q;
    const __half* bias;
    const float* scale;
    int* status;
    // stream-K (conv_streamk_kernel): the k-blocks of all tiles form one sequence of sk_units = tiles * kblocks units
    // that is cut into gridDim.x equal runs; a tile whose k-blocks fall into several runs is finished by the CTA that
    // holds its first k-block, the others hand their fp32 partial tile over through sk_part (one [128][BN] slot per
    // CTA) and sk_flags (one counter per slot, back at zero when the kernel ends).
    // per-image weights (1x1 stride-1 only): w is [N][K][C], image n uses its own [K][C] block; an m-tile is 128 pixels
    // of ONE image (wb_tpi tiles per image), activations / residual / output are addressed as (channel, pixel, image)
    int wb, wb_tpi;
    FastDiv div_tpi;
    int sk;
    int gsg, gsk;  // grouped convolution: input / output channels per super-group (0: dense), see conv2d_launch
    FastDiv div_gsk;
    int hints;     // L2 eviction hints: bit 0 input is dead after this layer, bit 1 residual is, bit 2 keep the output
    int rev;       // walk the m-tiles from the last to the first (see fvm_conv2d_f16_tile)
    int pair;      // conv_pair_kernel: two CTAs per tile of 256 pixels x BN channels (m_tiles counts 256-pixel tiles)
    uint32_t sk_units;
    FastDiv div_kb;
    float* sk_part;
    int* sk_flags;
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

// Epilogue arithmetic for one 32-column chunk of one output row: accumulator + bias (* scale) (+ residual) ->
// activation -> fp16, combined in place with the staged residual chunk. `stage_row` points at this row inside the
// 64-channel staging sub-tile (128-byte swizzle: 16-byte chunk index XOR (row & 7)); `bias_s` at the chunk's bias.
// ACT: 0 none, 1 relu, 3 silu, 5 gelu (erf), 2 = read p.act at run time. All loads are issued before the arithmetic.
// `part` / `nparts` / `part_stride` (stream-K only): fp32 partial sums of this row and these columns from `nparts` other
// CTAs (`part` points at this row's float4 of the chunk's first four columns in the first slot, slots are `part_stride`
// floats apart), added to the accumulator in that order before the epilogue arithmetic.
template <int ACT, bool RES, int W>
__device__ __forceinline__ void epilogue_chunk(const ConvParams& p, uint32_t taddr, uint32_t stage_row, uint32_t ch0,
                                               uint32_t row_xor, uint32_t bias_s, int n, int left,
                                               const float* part = nullptr, int nparts = 0, size_t part_stride = 0) {
    static_assert(W == 32 || W == 16, "chunks of 32 or 16 columns");
    uint32_t v[W];
    __syncwarp();
    // in flight while the bias and residual chunks are fetched from shared memory
    if constexpr (W == 32) tmem_ld_32x32b_x32(taddr, v);
    else tmem_ld_32x32b_x16(taddr, v);
    uint4 rw[W / 8];
    if (RES) {
#pragma unroll
        for (int j = 0; j < W / 8; ++j) rw[j] = lds128(stage_row + (((ch0 + j) ^ row_xor) << 4));
    }
    tmem_ld_wait();
    for (int q = 0; q < nparts; ++q) {
        // slot layout: [column / 4][row] float4, so that the 32 rows of a warp read (and wrote) 512 contiguous bytes
        const float4* src = reinterpret_cast<const float4*>(part + static_cast<size_t>(q) * part_stride);
#pragma unroll
        for (int i = 0; i < W / 4; ++i) {
            const float4 t = __ldcg(src + i * BM);  // written by another SM during this launch: read past L1
            v[4 * i] = __float_as_uint(__uint_as_float(v[4 * i]) + t.x);
            v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + t.y);
            v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + t.z);
            v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + t.w);
        }
    }
#pragma unroll
    for (int j = 0; j < W / 8; ++j) {
        if (8 * j < left) {
            const uint32_t r4[4] = {rw[j].x, rw[j].y, rw[j].z, rw[j].w};
            uint32_t o[4];
            unsigned long long bw[4];     // 8 fp32 bias values as 4 pairs
            lds_2xf2(bias_s + 32u * j, bw[0], bw[1]);
            lds_2xf2(bias_s + 32u * j + 16u, bw[2], bw[3]);
            if (ACT != 2 && p.scale == nullptr) {
                // fast path: packed fp32 adds; relu on the packed fp16 result (it commutes with the rounding); SiLU and
                // GELU in fp32 with the activation known at compile time
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    unsigned long long t = f2_add(f2_pack(v[8 * j + 2 * k], v[8 * j + 2 * k + 1]), bw[k]);
                    if (RES) t = f2_add(t, h2_to_f2(r4[k]));
                    if (ACT == 3) {
                        o[k] = f2_to_h2(f2_silu(t));
                    } else if (ACT == 5) {
                        o[k] = f2_to_h2(f2_gelu_erf(t));
                    } else {
                        o[k] = f2_to_h2(t);
                        if (ACT == 1) o[k] = h2_relu(o[k]);
                    }
                }
            } else {
                float f[8];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float blo, bhi;
                    f2_unpack(bw[k], blo, bhi);
                    f[2 * k] = __uint_as_float(v[8 * j + 2 * k]) + blo;
                    f[2 * k + 1] = __uint_as_float(v[8 * j + 2 * k + 1]) + bhi;
                }
                if (p.scale) {
                    const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.scale + n + 8 * j));
                    const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.scale + n + 8 * j + 4));
                    f[0] *= s0.x; f[1] *= s0.y; f[2] *= s0.z; f[3] *= s0.w;
                    f[4] *= s1.x; f[5] *= s1.y; f[6] *= s1.z; f[7] *= s1.w;
                }
                if (RES) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 t = unpack_h2(r4[k]);
                        f[2 * k] += t.x;
                        f[2 * k + 1] += t.y;
                    }
                }
                const int act = ACT == 2 ? p.act : ACT;
#pragma unroll
                for (int k = 0; k < 8; ++k) f[k] = act_f(f[k], act);
#pragma unroll
                for (int k = 0; k < 4; ++k) o[k] = pack_h2(f[2 * k], f[2 * k + 1]);
            }
            sts128(stage_row + (((ch0 + j) ^ row_xor) << 4), make_uint4(o[0], o[1], o[2], o[3]));
        }
    }
}

// This thread's row of one tile, the 32-column chunks of its epilogue group (group, group + 4, ..). BN is a multiple
// of 32, so every TMEM read is a full 32-column load inside the accumulator buffer.
template <int ACT, bool RES, int W>
__device__ __forceinline__ void epilogue_cols(const ConvParams& p, uint32_t t_row, uint32_t stage_row0, uint32_t row_xor,
                                              uint32_t bias_s, int n0, int ncols, int group) {
    for (int c0 = W * group; c0 < ncols; c0 += W * EPI_GROUPS) {
        const uint32_t sub = stage_row0 + static_cast<uint32_t>(c0 >> 6) * SUB_BYTES;
        epilogue_chunk<ACT, RES, W>(p, t_row + static_cast<uint32_t>(c0), sub, static_cast<uint32_t>((c0 & 63) >> 3), row_xor,
                                 bias_s + 4u * static_cast<uint32_t>(n0 + c0), n0 + c0, ncols - c0);
    }
}

// The chunk width (32 or 16 columns) is the one with which the busiest of the four groups has fewer columns to do:
// 16 for tiles of up to 64 columns and for widths like 144, 160 or 192 (5 or 6 chunks of 32 would leave one group
// with two chunks while the others have one).
template <int ACT, bool RES>
__device__ __forceinline__ void epilogue_rows(const ConvParams& p, uint32_t t_row, uint32_t stage_row0, uint32_t row_xor,
                                              uint32_t bias_s, int n0, int ncols, int group) {
    const int rounds32 = ((ncols + 31) / 32 + EPI_GROUPS - 1) / EPI_GROUPS;
    const int rounds16 = ((ncols + 15) / 16 + EPI_GROUPS - 1) / EPI_GROUPS;
    if (rounds16 * 16 < rounds32 * 32) epilogue_cols<ACT, RES, 16>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group);
    else epilogue_cols<ACT, RES, 32>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group);
}

// Tile number `it` of this CTA. Default: tiles blockIdx.x, blockIdx.x + gridDim.x, ... with the n-tile fastest.
// Weight-resident mode: the CTA owns n-tile (blockIdx.x % n_tiles) and walks m-tiles with stride gridDim.x / n_tiles
// (the grid is a multiple of n_tiles).
__device__ __forceinline__ bool tile_at(const ConvParams& p, int it, int& m_tile, int& n_tile) {
    if (p.bres) {
        const int q = static_cast<int>(fastdiv(blockIdx.x, p.div_ntiles));
        n_tile = static_cast<int>(blockIdx.x) - q * p.n_tiles;
        m_tile = q + it * static_cast<int>(fastdiv(gridDim.x, p.div_ntiles));
        if (m_tile >= p.m_tiles) return false;
        if (p.rev) m_tile = p.m_tiles - 1 - m_tile;
        return true;
    }
    const int tile = static_cast<int>(blockIdx.x) + it * static_cast<int>(gridDim.x);
    if (tile >= p.m_tiles * p.n_tiles) return false;
    m_tile = static_cast<int>(fastdiv(static_cast<uint32_t>(tile), p.div_ntiles));
    n_tile = tile - m_tile * p.n_tiles;
    if (p.rev) m_tile = p.m_tiles - 1 - m_tile;
    return true;
}

// Number of tiles tile_at() yields for this CTA.
__device__ __forceinline__ int cta_tile_count(const ConvParams& p) {
    if (p.bres) {
        const int per_n = static_cast<int>(fastdiv(gridDim.x, p.div_ntiles));
        const int q = static_cast<int>(fastdiv(blockIdx.x, p.div_ntiles));
        return q < p.m_tiles ? (p.m_tiles - q + per_n - 1) / per_n : 0;
    }
    const int tiles = p.m_tiles * p.n_tiles;
    return static_cast<int>(blockIdx.x) < tiles ? (tiles - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
}

// Shared memory map (after rounding the base up to 1024 bytes):
//   [stages x (A tile 16 KB | B tile BN*128 B)] [nepi x nsub x 16 KB staging] [barriers] [tmem slot, abort flag]
//   [bias copy, fp32, zero-padded to n_tiles*BN]
// Staging sub-tiles use the same 128-byte swizzle as the TMA maps of the residual and the output, so the residual
// arrives by TMA load, is combined in place by the epilogue threads (one row each, conflict-free 16-byte accesses)
// and leaves by TMA store: every byte of global traffic of this kernel is a bulk copy.
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_r, const __grid_constant__ CUtensorMap tmap_y,
                    const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_kb_bytes = static_cast<uint32_t>(p.BN) * BK * 2;          // one k-block of a weight tile
    const uint32_t b_stage_bytes = (p.tapk || p.bres) ? 0u : b_kb_bytes;
    const uint32_t a_stage_bytes = p.halo ? 0u : static_cast<uint32_t>(p.mt) * A_STAGE_BYTES;
    const uint32_t stage_bytes = a_stage_bytes + b_stage_bytes;
    const int tpk = p.tapk ? BK / p.tapk : 0;                                  // taps per k-block (8 or 4)
    const uint32_t tap_sub_bytes = static_cast<uint32_t>(BM * p.tapk * 2);    // one tap of one 128-pixel sub-tile
    const uint32_t tap_a_bytes = static_cast<uint32_t>(p.mt) * tap_sub_bytes;  // one tap of all sub-tiles of a stage
    // tap-packed mode: all weights of the (single) n-tile stay resident: one [BN x 16 B] block per tap
    const uint32_t tap_b_bytes = static_cast<uint32_t>(p.BN * p.tapk * 2);
    const uint32_t bres_base = smem_base + static_cast<uint32_t>(p.stages) * stage_bytes;
    const uint32_t stem_b_bytes = static_cast<uint32_t>(p.BN) * 16u;          // stem mode: one tap of the weights, [BN][8]
    const uint32_t bres_bytes = p.tapk ? static_cast<uint32_t>(p.kblocks * tpk) * tap_b_bytes
                                : p.halo == 2 ? static_cast<uint32_t>(p.stem_taps) * stem_b_bytes
                                : (p.bres ? static_cast<uint32_t>(p.kblocks) * b_kb_bytes : 0u);
    const uint32_t halo_base = bres_base + bres_bytes;
    const uint32_t halo_bytes = p.hbytes;
    const uint32_t epi_base = halo_base + static_cast<uint32_t>(p.nh) * halo_bytes;
    const uint32_t epi_bytes = static_cast<uint32_t>(p.mt * p.nsub) * SUB_BYTES;   // staging: [mt][nsub] sub-tiles
    const uint32_t bar_base = epi_base + static_cast<uint32_t>(p.nepi) * epi_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + MAX_ACC + a); };
    auto res_full_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + e); };
    auto epi_done_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + MAX_EPI + e); };
    auto epi_free_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + 2 * MAX_EPI + e); };
    const uint32_t bres_full_bar = bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + 3 * MAX_EPI);
    auto hfull_bar = [&](int h) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + 3 * MAX_EPI + 1 + h); };
    auto hempty_bar = [&](int h) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + 3 * MAX_EPI + 1 + MAX_HALO + h); };
    const uint32_t misc_off = (bar_base - smem_u32(smem_raw)) + 8u * NUM_BARRIERS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + misc_off + 4);
    // bar_base is 1024-aligned; the barrier block plus MISC_BYTES (tmem slot, abort flag, padding) is a multiple of 16:
    // the bias copy that follows is 16-byte aligned, as its 128-bit shared loads require
    static_assert((8 * NUM_BARRIERS + MISC_BYTES) % 16 == 0, "bias copy must be 16-byte aligned");
    const uint32_t bias_off = misc_off + MISC_BYTES;
    const uint32_t bias_base = smem_u32(smem_raw) + bias_off;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // warp-uniform by construction
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < p.nacc; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), EPI_WARPS);   // one arrival per epilogue warp
        }
        for (int e = 0; e < p.nepi; ++e) {
            mbar_init(res_full_bar(e), 1);
            mbar_init(epi_done_bar(e), EPI_WARPS);
            mbar_init(epi_free_bar(e), 1);
        }
        mbar_init(bres_full_bar, 1);
        for (int h = 0; h < p.nh; ++h) {
            mbar_init(hfull_bar(h), 1);
            mbar_init(hempty_bar(h), 1);
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
    // Everything above touches only this CTA's shared memory / TMEM. Programmatic dependent launch: this grid may have
    // been started while its predecessor was still draining, so the two threads that touch activations or outputs
    // (the producer before its first activation / residual load, the store thread before its first store) wait for
    // the preceding kernels with griddepcontrol.wait; weights and bias are constants and are fetched before that.
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // One elected lane runs the whole role and issues every bulk load (issuing from several lanes of a warp makes
        // the compiler serialise them anyway, at a higher cost per load).
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int e = 0;
            uint32_t e_phase = 0;   // one parity bit per staging buffer
            bool ok = true;
            const int PQ = p.P * p.Q;
            auto load_w = [&](uint32_t dst, uint32_t bar, int c0, int c1, int c2) {
                tma_load_3d(dst, &tmap_b, bar, c0, c1, c2);
            };
            const unsigned long long pol_a = (p.hints & 1) ? l2_policy_evict_first() : 0ull;
            const unsigned long long pol_r = (p.hints & 2) ? l2_policy_evict_first() : 0ull;
            if (p.tapk) {
                // weights of every tap (taps past R*S are out of bounds of the weight tensor: zero-filled)
                mbar_expect_tx(bres_full_bar, bres_bytes);
                for (int t = 0; t < p.kblocks * tpk; ++t)
                    load_w(bres_base + static_cast<uint32_t>(t) * tap_b_bytes, bres_full_bar, 0, t, 0);
            }
            int m_tile, n_tile;
            if (p.halo == 2) {
                // stem mode: every tap's [BN][8] block (taps past R*S are out of bounds of the weight tensor: zeros)
                mbar_expect_tx(bres_full_bar, bres_bytes);
                for (int t = 0; t < p.stem_taps; ++t)
                    load_w(bres_base + static_cast<uint32_t>(t) * stem_b_bytes, bres_full_bar, 0, t, 0);
            } else if (p.bres && tile_at(p, 0, m_tile, n_tile)) {
                // this CTA's weight tile, all k-blocks, once: k-block kb = (tap kb / cchunks, channels (kb % cchunks)*64)
                mbar_expect_tx(bres_full_bar, bres_bytes);
                int tp = 0, cc = 0;
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    load_w(bres_base + static_cast<uint32_t>(kb) * b_kb_bytes, bres_full_bar, cc * BK, tp,
                                n_tile * p.BN);
                    if (++cc == p.cchunks) { cc = 0; ++tp; }
                }
            }
            // Streamed weights: the B tiles of the first k-blocks (one per pipeline stage) are requested before the wait
            // as well; their barriers are armed for the whole stage, the A tiles follow after the wait.
            int pre = 0;
            if (!p.tapk && !p.bres && !p.halo && !p.wb) {
                for (int pit = 0; pre < p.stages && tile_at(p, pit, m_tile, n_tile); ++pit) {
                    int tap = 0, cc = 0;
                    for (int kb = 0; kb < p.kblocks && pre < p.stages; ++kb, ++pre) {
                        mbar_expect_tx(full_bar(pre), stage_bytes);
                        load_w(smem_base + static_cast<uint32_t>(pre) * stage_bytes + a_stage_bytes, full_bar(pre), cc * BK, tap, n_tile * p.BN);
                        if (++cc == p.cchunks) { cc = 0; ++tap; }
                    }
                }
            }
            int issued = 0;       // k-blocks issued so far (the first `pre` have their barrier armed and B on the way)
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int hs = 0;
            uint32_t hphase = 0;
            for (int pit = 0; ok && tile_at(p, pit, m_tile, n_tile); ++pit) {
                const int m0 = m_tile * BM * p.mt;
                const int n0 = n_tile * p.BN;
                int wb_img = 0, wb_row0 = 0;      // per-image weights: m_tile = (image, 128-pixel tile of that image)
                if (p.wb) {
                    wb_img = static_cast<int>(fastdiv(static_cast<uint32_t>(m_tile), p.div_tpi));
                    wb_row0 = (m_tile - wb_img * p.wb_tpi) * BM * p.mt;
                }
                // grouped convolution: the input channels of this n-tile's super-group start at goff
                const int goff = p.gsg ? static_cast<int>(fastdiv(static_cast<uint32_t>(n0), p.div_gsk)) * p.gsg : 0;
                // halo mode: m_tile = (image, patch row, patch column)
                int himg = 0, hy0 = 0, hx0 = 0;
                if (p.halo) {
                    himg = static_cast<int>(fastdiv(static_cast<uint32_t>(m_tile), p.div_txy));
                    const int rem = m_tile - himg * p.tiles_x * p.tiles_y;
                    const int ty = static_cast<int>(fastdiv(static_cast<uint32_t>(rem), p.div_tx));
                    hy0 = ty * HALO_TH;
                    hx0 = (rem - ty * p.tiles_x) * HALO_TW;
                }
                if (p.has_res) {
                    // residual tile of this output tile -> staging buffer e (free once its previous store was read out)
                    if (!mbar_wait(epi_free_bar(e), ((e_phase >> e) & 1u) ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    e_phase ^= 1u << e;
                    const int nsub = min(p.nsub, (p.K - n0 + 63) >> 6);
                    mbar_expect_tx(res_full_bar(e), static_cast<uint32_t>(p.mt * nsub) * SUB_BYTES);
                    for (int mt = 0; mt < p.mt; ++mt)
                        for (int sub = 0; sub < nsub; ++sub) {
                            const uint32_t dst = epi_base + static_cast<uint32_t>(e) * epi_bytes +
                                                 static_cast<uint32_t>(mt * p.nsub + sub) * SUB_BYTES;
                            if (p.halo) tma_load_4d(dst, &tmap_r, res_full_bar(e), n0 + sub * 64, hx0, hy0, himg, pol_r);
                            else if (p.wb) tma_load_3d(dst, &tmap_r, res_full_bar(e), n0 + sub * 64, wb_row0 + mt * BM, wb_img);
                            else tma_load_2d(dst, &tmap_r, res_full_bar(e), n0 + sub * 64, m0 + mt * BM, pol_r);
                        }
                    if (++e == p.nepi) e = 0;
                }
                if (p.halo) {
                    // per 64-channel chunk: one staged input patch (rows hy0-ph .., 16 pixels from hx0-pw, zero outside
                    // the image), then the 9 weight tiles of that chunk through the stage ring (unless resident)
                    for (int hc = 0; ok && hc < p.cchunks; ++hc) {
                        if (!mbar_wait(hempty_bar(hs), hphase ^ 1u, abort_flag)) {
                            atomicExch(p.status, STATUS_WAIT_PRODUCER);
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(hfull_bar(hs), p.htx);
                        if (p.halo == 2)     // (channel, plane column, plane, input row, image)
                            tma_load_5d(halo_base + static_cast<uint32_t>(hs) * halo_bytes, &tmap_a, hfull_bar(hs), 0,
                                        hx0 + p.stem_xlo, 0, 2 * hy0 - p.ph, himg);
                        else
                            tma_load_4d(halo_base + static_cast<uint32_t>(hs) * halo_bytes, &tmap_a, hfull_bar(hs), goff + hc * BK,
                                        hx0 - p.pw, hy0 - p.ph, himg, pol_a);
                        if (++hs == p.nh) { hs = 0; hphase ^= 1u; }
                        if (p.bres) continue;
                        for (int tp = 0; tp < p.taps; ++tp) {
                            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                                atomicExch(p.status, STATUS_WAIT_PRODUCER);
                                ok = false;
                                break;
                            }
                            mbar_expect_tx(full_bar(stage), stage_bytes);
                            load_w(smem_base + static_cast<uint32_t>(stage) * stage_bytes, full_bar(stage),
                                        hc * BK, tp, n0);
                            if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                        }
                    }
                    continue;
                }
                int img = 0, h0 = 0, w0 = 0;
                if (p.im2col) {
                    img = static_cast<int>(fastdiv(static_cast<uint32_t>(m0), p.div_pq));
                    const int rem = m0 - img * PQ;
                    const int pp = static_cast<int>(fastdiv(static_cast<uint32_t>(rem), p.div_q));
                    const int qq = rem - pp * p.Q;
                    h0 = pp * p.sh - p.ph;
                    w0 = qq * p.sw - p.pw;
                }
                int tap = 0, cc = 0, r = 0, s = 0;
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    const bool armed = issued < pre;      // this stage's barrier and B tile were set up before the wait
                    ++issued;
                    if (!armed && !mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + static_cast<uint32_t>(stage) * stage_bytes;
                    const uint32_t b_dst = a_dst + a_stage_bytes;
                    if (!armed) mbar_expect_tx(full_bar(stage), stage_bytes);
                    if (p.tapk) {
                        // 8 (or 4) taps of 8 (16) channels: each lands as a dense [128*mt pixels][16 (32) B] block. Taps
                        // past the filter re-read the last tap; their weights are zero.
                        for (int j = 0; j < tpk; ++j) {
                            const int t = min(kb * tpk + j, p.taps - 1);
                            const int tr = t / p.S, ts = t - tr * p.S;
                            tma_load_im2col_4d(a_dst + static_cast<uint32_t>(j) * tap_a_bytes, &tmap_a, full_bar(stage), 0,
                                               w0, h0, img, static_cast<uint16_t>(ts * p.dw),
                                               static_cast<uint16_t>(tr * p.dh));
                        }
                        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    if (!p.bres && !armed) load_w(b_dst, full_bar(stage), cc * BK, tap, n0 + wb_img * p.K);
                    if (p.im2col) {
                        tma_load_im2col_4d(a_dst, &tmap_a, full_bar(stage), goff + cc * BK, w0, h0, img,
                                           static_cast<uint16_t>(s * p.dw), static_cast<uint16_t>(r * p.dh), pol_a);
                    } else if (p.wb) {
                        tma_load_3d(a_dst, &tmap_a, full_bar(stage), cc * BK, wb_row0, wb_img);
                    } else {
                        for (int l = 0; l < p.a_loads; ++l)
                            tma_load_2d(a_dst + static_cast<uint32_t>(l * p.a_rows) * 128u, &tmap_a, full_bar(stage),
                                        goff + cc * BK, m0 + l * p.a_rows, pol_a);
                    }
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
                for (int i = 0; i < p.nh; ++i) {
                    if (!mbar_wait(hempty_bar(hs), hphase ^ 1u, abort_flag)) break;
                    if (++hs == p.nh) { hs = 0; hphase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        // One elected lane runs the whole role. Every loop bound and branch of the role depends on kernel parameters
        // and counters only (a wait that runs out is recorded and the role carries on: once the abort flag is up all
        // waits of the CTA return at once), so the compiler can keep the counters and descriptors in uniform
        // registers, which the tcgen05 instructions read their operands from; measured, this halves the issue cost.
        // Descriptors are kept as 32-bit low words (start address) that advance by constants; the high words (stride,
        // version, swizzle) never change; the four MMAs of a k-block are one instruction sequence.
        if (elect_one()) {
            const uint32_t idesc = umma_idesc_f16_f32(BM, p.BN);
            const uint32_t hi128 = static_cast<uint32_t>(umma_desc_sw128(0) >> 32);
            const uint32_t hi_halo = static_cast<uint32_t>(umma_desc_sw128_at(0, HALO_PITCH * 128u) >> 32);
            auto lo_of = [](uint32_t addr) { return ((addr & 0x3ffffu) >> 4) | 0x10000u; };
            const uint32_t stage_step = stage_bytes >> 4;
            const uint32_t a_lo0 = lo_of(smem_base);
            const int my_tiles = cta_tile_count(p);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t st_lo = a_lo0;   // low descriptor word of the current stage's first byte
            uint32_t acc_phase = 0;   // one parity bit per accumulator buffer
            int acc = -1;
            bool failed = false;
            int mma_hs = 0;
            uint32_t mma_hphase = 0;
#define NEXT_STAGE()                                                          \
    do {                                                                      \
        st_lo += stage_step;                                                  \
        if (++stage == p.stages) { stage = 0; phase ^= 1u; st_lo = a_lo0; }   \
    } while (0)
            if ((p.tapk || p.bres) && my_tiles > 0) failed |= !mbar_wait(bres_full_bar, 0u, abort_flag);
            // Look-ahead: the barrier of the next step (stage, staged patch, accumulator) is tested while the MMAs of
            // the current step are issued; the blocking wait runs only if that test said "not yet".
            uint32_t st_ready = 0, acc_ready = 0, h_ready = 0;
            for (int it = 0; it < my_tiles; ++it) {
                if (++acc == p.nacc) acc = 0;
                if (!acc_ready) failed |= !mbar_wait(tempty_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag);
                acc_phase ^= 1u << acc;
                const int acc_next = acc + 1 == p.nacc ? 0 : acc + 1;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.acc_stride);
                if (p.halo == 2) {
                    // Stem mode. Output pixel (oy, ox) of the patch, tap (r, s): input row 2*oy + r, plane (s - pw) & 1,
                    // plane column ox + (s - pw - plane) / 2. One MMA (K = 16) covers taps (r, s) and (r + 1, s): its two
                    // K halves are one staged row apart (LBO), its 8-pixel groups (one output row each) two staged rows
                    // (SBO); no swizzle. Weights: tap blocks [BN][8]; the K halves are S blocks apart.
                    if (!h_ready) failed |= !mbar_wait(hfull_bar(mma_hs), mma_hphase, abort_flag);
                    tc_fence_after();
                    {
                        const bool hwrap = mma_hs + 1 == p.nh;
                        h_ready = mbar_test(hfull_bar(hwrap ? 0 : mma_hs + 1), hwrap ? mma_hphase ^ 1u : mma_hphase);
                        acc_ready = mbar_test(tempty_bar(acc_next), ((acc_phase >> acc_next) & 1u) ^ 1u);
                    }
                    const uint32_t prow16 = p.stem_prow >> 4, pplane16 = p.stem_prow >> 5;
                    const uint32_t a_hi = (2u * prow16) | (1u << 14);                 // SBO, descriptor version
                    const uint32_t b_hi = (128u >> 4) | (1u << 14);
                    const uint32_t a_base = (((halo_base + static_cast<uint32_t>(mma_hs) * halo_bytes) & 0x3ffffu) >> 4) | (prow16 << 16);
                    const uint32_t b_base = ((bres_base & 0x3ffffu) >> 4) | ((static_cast<uint32_t>(p.S) * (stem_b_bytes >> 4)) << 16);
                    const int rpairs = p.stem_taps / (2 * p.S);
                    uint32_t first = 0;
                    for (int ts = 0; ts < p.S; ++ts) {
                        const int d = ts - p.pw, par = d & 1;
                        uint32_t a_lo = a_base + static_cast<uint32_t>(par) * pplane16 + static_cast<uint32_t>(((d - par) >> 1) - p.stem_xlo);
                        uint32_t b_lo = b_base + static_cast<uint32_t>(ts) * (stem_b_bytes >> 4);
                        const uint32_t b_step = 2u * static_cast<uint32_t>(p.S) * (stem_b_bytes >> 4);
                        if (rpairs == 4) {       // 7- and 8-row filters: the column's four tap pairs as one sequence
                            umma_f16_stepped4(d_tmem, a_lo, a_hi, 2u * prow16, b_lo, b_hi, b_step, idesc, first);
                            first = 1;
                            continue;
                        }
                        for (int rp = 0; rp < rpairs; ++rp) {
                            umma_f16_words(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, first);
                            first = 1;
                            a_lo += 2u * prow16;
                            b_lo += b_step;
                        }
                    }
                    umma_commit(hempty_bar(mma_hs));
                    if (++mma_hs == p.nh) { mma_hs = 0; mma_hphase ^= 1u; }
                    umma_commit(tfull_bar(acc));
                    continue;
                }
                if (p.halo) {
                    for (int hc = 0; hc < p.cchunks; ++hc) {
                        if (!h_ready) failed |= !mbar_wait(hfull_bar(mma_hs), mma_hphase, abort_flag);
                        tc_fence_after();
                        // tap (tr, ts): the A rows are the staged patch shifted by (tr, ts) * dilation pixels; 8-pixel
                        // groups (one patch row each) are one staged row (16 pixels = 2 KB) apart. The swizzle phase
                        // follows the absolute shared-memory address, so a start at any 128-byte row needs no base offset.
                        uint32_t b_lo_res = lo_of(bres_base + static_cast<uint32_t>(hc) * b_kb_bytes);
                        uint32_t row_lo = lo_of(halo_base + static_cast<uint32_t>(mma_hs) * halo_bytes);
#pragma unroll
                        for (int tr = 0; tr < 3; ++tr) {        // halo mode is 3x3 only: straight-line code for the 9 taps
                            uint32_t a_lo = row_lo;
#pragma unroll
                            for (int ts = 0; ts < 3; ++ts) {
                                uint32_t b_lo = b_lo_res;
                                if (!p.bres) {
                                    if (!st_ready) failed |= !mbar_wait(full_bar(stage), phase, abort_flag);
                                    tc_fence_after();
                                    const bool wrap = stage + 1 == p.stages;
                                    st_ready = mbar_test(full_bar(wrap ? 0 : stage + 1), wrap ? phase ^ 1u : phase);
                                    b_lo = st_lo;
                                }
                                if (tr == 2 && ts == 0) {     // before the last row of taps: look at the next patch / accumulator
                                    const bool hwrap = mma_hs + 1 == p.nh;
                                    h_ready = mbar_test(hfull_bar(hwrap ? 0 : mma_hs + 1), hwrap ? mma_hphase ^ 1u : mma_hphase);
                                    if (hc == p.cchunks - 1)
                                        acc_ready = mbar_test(tempty_bar(acc_next), ((acc_phase >> acc_next) & 1u) ^ 1u);
                                }
                                umma_f16_kblock(d_tmem, a_lo, hi_halo, b_lo, hi128, idesc, static_cast<uint32_t>((hc | tr | ts) != 0));
                                if (!p.bres) {
                                    umma_commit(empty_bar(stage));
                                    NEXT_STAGE();
                                }
                                a_lo += static_cast<uint32_t>(p.dw) * 8u;                          // next tap: dw pixels of 128 B
                                b_lo_res += static_cast<uint32_t>(p.cchunks) * (b_kb_bytes >> 4);  // resident: next tap's block
                            }
                            row_lo += static_cast<uint32_t>(p.dh * HALO_PITCH) * 8u;
                        }
                        umma_commit(hempty_bar(mma_hs));     // the staged patch is free once these MMAs have read it
                        if (++mma_hs == p.nh) { mma_hs = 0; mma_hphase ^= 1u; }
                    }
                    umma_commit(tfull_bar(acc));
                    continue;
                }
                uint32_t bres_lo = lo_of(bres_base);
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!st_ready) failed |= !mbar_wait(full_bar(stage), phase, abort_flag);
                    tc_fence_after();
                    {
                        const bool wrap = stage + 1 == p.stages;
                        st_ready = mbar_test(full_bar(wrap ? 0 : stage + 1), wrap ? phase ^ 1u : phase);
                    }
                    if (kb == p.kblocks - 1)
                        acc_ready = mbar_test(tempty_bar(acc_next), ((acc_phase >> acc_next) & 1u) ^ 1u);
                    const uint32_t a_src = smem_base + static_cast<uint32_t>(stage) * stage_bytes;
                    if (p.tapk == 16) {
                        // one MMA (K = 16) per tap: rows of 32 bytes in the 32-byte-swizzled layout
                        for (int mt = 0; mt < p.mt; ++mt) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const uint64_t a_desc = umma_desc_sw32(a_src + static_cast<uint32_t>(k) * tap_a_bytes +
                                                                       static_cast<uint32_t>(mt) * tap_sub_bytes);
                                const uint64_t b_desc =
                                    umma_desc_sw32(bres_base + static_cast<uint32_t>(kb * 4 + k) * tap_b_bytes);
                                umma_f16(d_tmem + static_cast<uint32_t>(mt * p.BN), a_desc, b_desc, idesc,
                                         (kb | k) != 0 ? 1u : 0u);
                            }
                        }
                    } else if (p.tapk) {
                        // K = 16 spans two taps: the two 16-byte K halves are one tap block apart (LBO); 8-row groups
                        // are 128 bytes apart (SBO); no swizzle
                        for (int mt = 0; mt < p.mt; ++mt) {
#pragma unroll
                            for (int k = 0; k < TAPS_PER_KBLOCK / 2; ++k) {
                                const uint64_t a_desc = umma_desc_interleaved(
                                    a_src + static_cast<uint32_t>(2 * k) * tap_a_bytes + static_cast<uint32_t>(mt) * tap_sub_bytes,
                                    tap_a_bytes, 128u);
                                const uint64_t b_desc = umma_desc_interleaved(
                                    bres_base + static_cast<uint32_t>(kb * TAPS_PER_KBLOCK + 2 * k) * tap_b_bytes, tap_b_bytes,
                                    128u);
                                umma_f16(d_tmem + static_cast<uint32_t>(mt * p.BN), a_desc, b_desc, idesc,
                                         (kb | k) != 0 ? 1u : 0u);
                            }
                        }
                    } else {
                        const uint32_t b_lo = p.bres ? bres_lo : st_lo + (a_stage_bytes >> 4);
                        bres_lo += b_kb_bytes >> 4;
                        // sub-tile mt: its own 128 rows of A, the shared B tile, accumulator columns [mt*BN, (mt+1)*BN)
                        for (int mt = 0; mt < p.mt; ++mt)
                            umma_f16_kblock(d_tmem + static_cast<uint32_t>(mt * p.BN),
                                            st_lo + static_cast<uint32_t>(mt) * (A_STAGE_BYTES >> 4), hi128, b_lo, hi128, idesc,
                                            static_cast<uint32_t>(kb != 0));
                    }
                    umma_commit(empty_bar(stage));   // frees the stage once these MMAs have read it
                    NEXT_STAGE();
                }
                umma_commit(tfull_bar(acc));  // accumulator complete
            }
#undef NEXT_STAGE
            if (failed) atomicExch(p.status, STATUS_WAIT_MMA);
        }
        __syncwarp();
    } else if (warp < STORE_WARP) {
        // ------------------------------------------------------------------ epilogue
        // EPI_GROUPS groups of 4 warps (one warp per TMEM lane group). All groups work on every tile: group g takes the
        // 32-column chunks g, g + 4, .. of the accumulator, so a tile is finished in a quarter of the time one group
        // would need (short tail at the end of the kernel, two accumulators and two or three staging buffers suffice).
        const int lane_group = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row = lane_group * 32 + lane;       // row of the tile = TMEM lane
        const uint32_t row_xor = static_cast<uint32_t>(row & 7);
        const uint32_t bias_s = bias_base;
        const uint32_t stage0 = epi_base + static_cast<uint32_t>(row) * 128u;
        {
            // fp32 copy of the bias (the epilogue adds it as packed pairs), filled by the epilogue warps only, off the
            // producer's and the MMA issuer's path; a named barrier over the 16 epilogue warps publishes it
            float* bias_f = reinterpret_cast<float*>(smem_raw + bias_off);
            for (int i = threadIdx.x - 64; i < p.bias_elems; i += EPI_WARPS * 32)
                bias_f[i] = (p.bias != nullptr && i < p.K) ? __half2float(p.bias[i]) : 0.f;
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        }
        uint32_t acc_phase = 0;   // one parity bit per accumulator buffer
        uint32_t e_phase = 0;     // one parity bit per staging buffer
        int e = 0;
        int acc = -1;
        int it = 0;
        bool ok = true;
        int m_tile, n_tile;
        for (; ok && tile_at(p, it, m_tile, n_tile); ++it) {
            if (++acc == p.nacc) acc = 0;
            const int n0 = n_tile * p.BN;
            // staging buffer: with a residual it is filled by TMA (res_full); without, wait until it is free
            const bool got_buf = p.has_res ? mbar_wait<EPI_BACKOFF_NS>(res_full_bar(e), (e_phase >> e) & 1u, abort_flag)
                                           : mbar_wait<EPI_BACKOFF_NS>(epi_free_bar(e), ((e_phase >> e) & 1u) ^ 1u, abort_flag);
            if (!got_buf || !mbar_wait<EPI_BACKOFF_NS>(tfull_bar(acc), (acc_phase >> acc) & 1u, abort_flag)) {
                if (lane == 0) atomicExch(p.status, STATUS_WAIT_EPILOGUE);
                ok = false;
                break;
            }
            e_phase ^= 1u << e;
            acc_phase ^= 1u << acc;
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                                   static_cast<uint32_t>(acc * p.acc_stride);
            const uint32_t stage_row0 = stage0 + static_cast<uint32_t>(e) * epi_bytes;
            const int ncols = min(p.BN, p.K - n0);   // multiple of 8
            // activation as a template argument for the common ones (0 none, 1 relu, 3 silu, 5 gelu-erf); 2 = read at run time
            const int act_t = (p.act == 0 || p.act == 1 || p.act == 3 || p.act == 5) ? p.act : 2;
            const int variant = act_t * 2 + (p.has_res ? 1 : 0);
            for (int mt = 0; mt < p.mt; ++mt) {
                const uint32_t t_sub = t_row + static_cast<uint32_t>(mt * p.BN);
                const uint32_t s_sub = stage_row0 + static_cast<uint32_t>(mt * p.nsub) * SUB_BYTES;
                switch (variant) {
                    case 0: epilogue_rows<0, false>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 1: epilogue_rows<0, true>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 2: epilogue_rows<1, false>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 3: epilogue_rows<1, true>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 4: epilogue_rows<2, false>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 5: epilogue_rows<2, true>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 6: epilogue_rows<3, false>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 7: epilogue_rows<3, true>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    case 10: epilogue_rows<5, false>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                    default: epilogue_rows<5, true>(p, t_sub, s_sub, row_xor, bias_s, n0, ncols, group); break;
                }
            }
            // all TMEM reads of this warp are done: hand the accumulator back; publish this warp's rows of the staged
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
        if (elect_one()) {
            uint32_t e_phase = 0;   // one parity bit per staging buffer
            int e = 0;
            const unsigned long long pol_y = (p.hints & 4) ? l2_policy_evict_last() : 0ull;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            int m_tile, n_tile;
            for (int sit = 0; ok && tile_at(p, sit, m_tile, n_tile); ++sit) {
                const int m0 = m_tile * BM * p.mt;
                const int n0 = n_tile * p.BN;
                if (!mbar_wait<EPI_BACKOFF_NS>(epi_done_bar(e), (e_phase >> e) & 1u, abort_flag)) {
                    atomicExch(p.status, STATUS_WAIT_STORE);
                    ok = false;
                    break;
                }
                e_phase ^= 1u << e;
                const int nsub = min(p.nsub, (p.K - n0 + 63) >> 6);
                if (p.halo) {
                    const int himg = static_cast<int>(fastdiv(static_cast<uint32_t>(m_tile), p.div_txy));
                    const int rem = m_tile - himg * p.tiles_x * p.tiles_y;
                    const int ty = static_cast<int>(fastdiv(static_cast<uint32_t>(rem), p.div_tx));
                    for (int sub = 0; sub < nsub; ++sub)      // 16 x 8 pixel patch, clipped at the image border
                        tma_store_4d(&tmap_y, epi_base + static_cast<uint32_t>(e) * epi_bytes + static_cast<uint32_t>(sub) * SUB_BYTES,
                                     n0 + sub * 64, (rem - ty * p.tiles_x) * HALO_TW, ty * HALO_TH, himg);
                }
                if (p.wb) {       // per-image weights: (channel, pixel of the image, image), clipped at the image's last pixel
                    const int wb_img = static_cast<int>(fastdiv(static_cast<uint32_t>(m_tile), p.div_tpi));
                    const int wb_row0 = (m_tile - wb_img * p.wb_tpi) * BM * p.mt;
                    for (int mt = 0; mt < p.mt && wb_row0 + mt * BM < p.P * p.Q; ++mt)
                        for (int sub = 0; sub < nsub; ++sub)
                            tma_store_3d(&tmap_y,
                                         epi_base + static_cast<uint32_t>(e) * epi_bytes +
                                             static_cast<uint32_t>(mt * p.nsub + sub) * SUB_BYTES,
                                         n0 + sub * 64, wb_row0 + mt * BM, wb_img);
                }
                for (int mt = 0; !p.halo && !p.wb && mt < p.mt && m0 + mt * BM < p.M; ++mt)     // sub-tiles past the last row: nothing to store
                    for (int sub = 0; sub < nsub; ++sub)
                        tma_store_2d(&tmap_y,
                                     epi_base + static_cast<uint32_t>(e) * epi_bytes +
                                         static_cast<uint32_t>(mt * p.nsub + sub) * SUB_BYTES,
                                     n0 + sub * 64, m0 + mt * BM, pol_y);
                tma_store_commit();
                tma_store_wait_read();          // the staging buffer has been read out: it may be refilled
                mbar_arrive(epi_free_bar(e));
                if (++e == p.nepi) e = 0;
            }
            // Shared memory must outlive the stores' reads of it; the writes themselves complete asynchronously and are
            // visible to the next kernel through the usual kernel-boundary ordering.
            tma_store_wait_read();
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

// ------------------------------------------------------------------------------------------------ stream-K variant
// For layers with fewer tiles than SMs, or a ragged last wave (every 14x14 / 7x7 layer of a ResNet at batch 64, the
// classifier GEMM): the k-blocks of all tiles are laid end to end and every CTA takes an equal run of them, so all SMs
// pull the same share of the operands through their L2 ports whatever the tile count. A run covers the tail of one
// tile, whole tiles, and the head of another. A CTA that holds a tile's k-block 0 finishes the tile (bias, residual,
// activation, store); the CTAs holding its later k-blocks write their fp32 partial tile to their slot of p.sk_part and
// raise their counter in p.sk_flags. Because runs are contiguous, a partial tile is always the FIRST thing its CTA
// computes and the tile it is added to is the LAST thing the finishing CTA computes: no CTA waits for work that has not
// been started, and the wait (bounded like every other) is short. Counters return to zero by themselves: producers
// add EPI_WARPS, the finishing CTA's warps add EPI_WARPS more once they have read the slot, the last one resets it.
// Plain mode only: A by tiled or im2col TMA, B streamed per k-block, one 128-pixel sub-tile. Same roles and
// shared-memory map as conv_tcgen05_kernel.
static constexpr int STATUS_WAIT_STREAMK = 0x106;

struct SkSeg {
    int m_tile, n_tile;
    int kb0, kb1;      // k-blocks [kb0, kb1) of the tile
    int kind;          // 0 whole tile; 1 partial tile handed over through this CTA's slot; 2 head of a tile: finishes it
    int nparts;        // kind 2: the next `nparts` CTAs hold the rest of the tile
};

__device__ __forceinline__ uint32_t sk_run_begin(const ConvParams& p, uint32_t cta) {
    return static_cast<uint32_t>((static_cast<unsigned long long>(cta) * p.sk_units) / gridDim.x);
}

// Next segment of this CTA's run [u, u1); advances u.
__device__ __forceinline__ bool sk_next(const ConvParams& p, uint32_t& u, uint32_t u1, SkSeg& s) {
    if (u >= u1) return false;
    const uint32_t tile = fastdiv(u, p.div_kb);
    const int kb0 = static_cast<int>(u - tile * static_cast<uint32_t>(p.kblocks));
    const int kb1 = min(p.kblocks, kb0 + static_cast<int>(u1 - u));
    s.m_tile = static_cast<int>(fastdiv(tile, p.div_ntiles));
    s.n_tile = static_cast<int>(tile) - s.m_tile * p.n_tiles;
    s.kb0 = kb0;
    s.kb1 = kb1;
    s.nparts = 0;
    if (kb0 > 0) {
        s.kind = 1;
    } else if (kb1 == p.kblocks) {
        s.kind = 0;
    } else {
        s.kind = 2;
        const uint32_t tile_end = (tile + 1u) * static_cast<uint32_t>(p.kblocks);
        for (uint32_t j = blockIdx.x + 1; j < gridDim.x && sk_run_begin(p, j) < tile_end; ++j) ++s.nparts;
    }
    u += static_cast<uint32_t>(kb1 - kb0);
    return true;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* ptr) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_streamk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_r, const __grid_constant__ CUtensorMap tmap_y,
                    const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_kb_bytes = static_cast<uint32_t>(p.BN) * BK * 2;
    const uint32_t stage_bytes = A_STAGE_BYTES + b_kb_bytes;
    const uint32_t epi_base = smem_base + static_cast<uint32_t>(p.stages) * stage_bytes;
    const uint32_t epi_bytes = static_cast<uint32_t>(p.nsub) * SUB_BYTES;
    const uint32_t bar_base = epi_base + static_cast<uint32_t>(p.nepi) * epi_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + MAX_ACC + a); };
    auto res_full_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + e); };
    auto epi_done_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + MAX_EPI + e); };
    auto epi_free_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + 2 * MAX_EPI + e); };
    const uint32_t misc_off = (bar_base - smem_u32(smem_raw)) + 8u * NUM_BARRIERS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + misc_off + 4);
    const uint32_t bias_off = misc_off + MISC_BYTES;
    const uint32_t bias_base = smem_u32(smem_raw) + bias_off;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < p.nacc; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), EPI_WARPS);
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
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t run_begin = sk_run_begin(p, blockIdx.x), run_end = sk_run_begin(p, blockIdx.x + 1);
    const size_t slot_floats = static_cast<size_t>(BM) * p.BN;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int e = 0;
            uint32_t e_phase = 0;
            bool ok = true;
            const int PQ = p.P * p.Q;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t u = run_begin;
            SkSeg sg;
            while (ok && sk_next(p, u, run_end, sg)) {
                const int m0 = sg.m_tile * BM;
                const int n0 = sg.n_tile * p.BN;
                if (p.has_res && sg.kind != 1) {
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
                    img = static_cast<int>(fastdiv(static_cast<uint32_t>(m0), p.div_pq));
                    const int rem = m0 - img * PQ;
                    const int pp = static_cast<int>(fastdiv(static_cast<uint32_t>(rem), p.div_q));
                    const int qq = rem - pp * p.Q;
                    h0 = pp * p.sh - p.ph;
                    w0 = qq * p.sw - p.pw;
                }
                int tap = sg.kb0 / p.cchunks;
                int cc = sg.kb0 - tap * p.cchunks;
                int r = tap / p.S;
                int s = tap - r * p.S;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + static_cast<uint32_t>(stage) * stage_bytes;
                    mbar_expect_tx(full_bar(stage), stage_bytes);
                    tma_load_3d(a_dst + A_STAGE_BYTES, &tmap_b, full_bar(stage), cc * BK, tap, n0);
                    if (p.im2col)
                        tma_load_im2col_4d(a_dst, &tmap_a, full_bar(stage), cc * BK, w0, h0, img,
                                           static_cast<uint16_t>(s * p.dw), static_cast<uint16_t>(r * p.dh));
                    else
                        tma_load_2d(a_dst, &tmap_a, full_bar(stage), cc * BK, m0);
                    if (++cc == p.cchunks) {
                        cc = 0;
                        ++tap;
                        if (++s == p.S) { s = 0; ++r; }
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (ok) {       // no bulk load of this CTA may be in flight when it exits
                for (int i = 0; i < p.stages; ++i) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) break;
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            const uint32_t idesc = umma_idesc_f16_f32(BM, p.BN);
            const uint32_t hi128 = static_cast<uint32_t>(umma_desc_sw128(0) >> 32);
            auto lo_of = [](uint32_t addr) { return ((addr & 0x3ffffu) >> 4) | 0x10000u; };
            const uint32_t stage_step = stage_bytes >> 4;
            const uint32_t a_lo0 = lo_of(smem_base);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t st_lo = a_lo0;
            uint32_t acc_phase = 0;
            int acc = -1;
            bool failed = false;
            uint32_t u = run_begin;
            SkSeg sg;
            while (sk_next(p, u, run_end, sg)) {
                if (++acc == p.nacc) acc = 0;
                failed |= !mbar_wait(tempty_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag);
                acc_phase ^= 1u << acc;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.acc_stride);
                for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
                    failed |= !mbar_wait(full_bar(stage), phase, abort_flag);
                    tc_fence_after();
                    umma_f16_kblock(d_tmem, st_lo, hi128, st_lo + (A_STAGE_BYTES >> 4), hi128, idesc,
                                    static_cast<uint32_t>(kb != sg.kb0));
                    umma_commit(empty_bar(stage));
                    st_lo += stage_step;
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; st_lo = a_lo0; }
                }
                umma_commit(tfull_bar(acc));
            }
            if (failed) atomicExch(p.status, STATUS_WAIT_MMA);
        }
        __syncwarp();
    } else if (warp < STORE_WARP) {
        // ------------------------------------------------------------------ epilogue
        const int lane_group = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row = lane_group * 32 + lane;
        const uint32_t row_xor = static_cast<uint32_t>(row & 7);
        const uint32_t bias_s = bias_base;
        const uint32_t stage0 = epi_base + static_cast<uint32_t>(row) * 128u;
        {
            float* bias_f = reinterpret_cast<float*>(smem_raw + bias_off);
            for (int i = threadIdx.x - 64; i < p.bias_elems; i += EPI_WARPS * 32)
                bias_f[i] = (p.bias != nullptr && i < p.K) ? __half2float(p.bias[i]) : 0.f;
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        }
        uint32_t acc_phase = 0, e_phase = 0;
        int e = 0, acc = -1;
        bool ok = true;
        uint32_t u = run_begin;
        SkSeg sg;
        const int act_t = (p.act == 0 || p.act == 1 || p.act == 3 || p.act == 5) ? p.act : 2;
        const int variant = act_t * 2 + (p.has_res ? 1 : 0);
        while (ok && sk_next(p, u, run_end, sg)) {
            if (++acc == p.nacc) acc = 0;
            const int n0 = sg.n_tile * p.BN;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                                   static_cast<uint32_t>(acc * p.acc_stride);
            if (sg.kind == 1) {
                // partial tile: fp32 accumulator rows to this CTA's slot, then the counter
                if (!mbar_wait<EPI_BACKOFF_NS>(tfull_bar(acc), (acc_phase >> acc) & 1u, abort_flag)) {
                    if (lane == 0) atomicExch(p.status, STATUS_WAIT_EPILOGUE);
                    ok = false;
                    break;
                }
                acc_phase ^= 1u << acc;
                tc_fence_after();
                float4* slot = reinterpret_cast<float4*>(p.sk_part + static_cast<size_t>(blockIdx.x) * slot_floats);
                for (int c0 = 32 * group; c0 < p.BN; c0 += 32 * EPI_GROUPS) {
                    uint32_t v[32];
                    __syncwarp();
                    tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c0), v);
                    tmem_ld_wait();
                    float4* dst = slot + static_cast<size_t>(c0 >> 2) * BM + row;      // [column / 4][row]
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        __stcg(dst + i * BM, make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                    __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3])));
                }
                __threadfence();                 // this thread's partial sums are visible device-wide before the counter moves
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(tempty_bar(acc));
                    atomicAdd(p.sk_flags + blockIdx.x, 1);
                }
                continue;
            }
            const bool got_buf = p.has_res ? mbar_wait<EPI_BACKOFF_NS>(res_full_bar(e), (e_phase >> e) & 1u, abort_flag)
                                           : mbar_wait<EPI_BACKOFF_NS>(epi_free_bar(e), ((e_phase >> e) & 1u) ^ 1u, abort_flag);
            if (!got_buf || !mbar_wait<EPI_BACKOFF_NS>(tfull_bar(acc), (acc_phase >> acc) & 1u, abort_flag)) {
                if (lane == 0) atomicExch(p.status, STATUS_WAIT_EPILOGUE);
                ok = false;
                break;
            }
            e_phase ^= 1u << e;
            acc_phase ^= 1u << acc;
            tc_fence_after();
            if (sg.kind == 2) {
                // the rest of this tile: wait (bounded) until every epilogue warp of each contributing CTA has written
                bool seen = true;
                if (lane == 0) {
                    for (int q = 0; q < sg.nparts && seen; ++q) {
                        const int* flag = p.sk_flags + blockIdx.x + 1 + q;
                        unsigned long long t0 = 0;
                        uint32_t spins = 0;
                        while (ld_acquire_gpu(flag) < EPI_WARPS) {
                            __nanosleep(64);
                            if ((++spins & 0x3f) == 0) {
                                const unsigned long long now = globaltimer_ns();
                                if (t0 == 0) t0 = now;
                                else if (*abort_flag || now - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; seen = false; break; }
                            }
                        }
                    }
                }
                seen = __shfl_sync(0xffffffffu, seen ? 1 : 0, 0) != 0;
                if (!seen) {
                    if (lane == 0) atomicExch(p.status, STATUS_WAIT_STREAMK);
                    ok = false;
                    break;
                }
            }
            const uint32_t stage_row0 = stage0 + static_cast<uint32_t>(e) * epi_bytes;
            const int ncols = min(p.BN, p.K - n0);
            const float* part_row = p.sk_part + static_cast<size_t>(blockIdx.x + 1) * slot_floats + static_cast<size_t>(row) * 4;
            for (int c0 = 32 * group; c0 < ncols; c0 += 32 * EPI_GROUPS) {
                const uint32_t sub = stage_row0 + static_cast<uint32_t>(c0 >> 6) * SUB_BYTES;
                const uint32_t ch0 = static_cast<uint32_t>((c0 & 63) >> 3);
                const uint32_t bs = bias_s + 4u * static_cast<uint32_t>(n0 + c0);
                const uint32_t ta = t_row + static_cast<uint32_t>(c0);
#define SK_CHUNK(A, R) epilogue_chunk<A, R, 32>(p, ta, sub, ch0, row_xor, bs, n0 + c0, ncols - c0, part_row + static_cast<size_t>(c0) * BM, sg.nparts, slot_floats)
                switch (variant) {
                    case 0: SK_CHUNK(0, false); break;
                    case 1: SK_CHUNK(0, true); break;
                    case 2: SK_CHUNK(1, false); break;
                    case 3: SK_CHUNK(1, true); break;
                    case 4: SK_CHUNK(2, false); break;
                    case 5: SK_CHUNK(2, true); break;
                    case 6: SK_CHUNK(3, false); break;
                    case 7: SK_CHUNK(3, true); break;
                    case 10: SK_CHUNK(5, false); break;
                    default: SK_CHUNK(5, true); break;
                }
#undef SK_CHUNK
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(tempty_bar(acc));
                mbar_arrive(epi_done_bar(e));
                // this warp has read the contributors' slots: EPI_WARPS more arrivals per counter, the last one clears it
                for (int q = 0; q < sg.nparts; ++q) {
                    int* flag = p.sk_flags + blockIdx.x + 1 + q;
                    if (atomicAdd(flag, 1) == 2 * EPI_WARPS - 1) atomicExch(flag, 0);
                }
            }
            if (++e == p.nepi) e = 0;
        }
    } else {
        // ------------------------------------------------------------------ store warp
        if (elect_one()) {
            uint32_t e_phase = 0;
            int e = 0;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            uint32_t u = run_begin;
            SkSeg sg;
            while (ok && sk_next(p, u, run_end, sg)) {
                if (sg.kind == 1) continue;
                const int m0 = sg.m_tile * BM;
                const int n0 = sg.n_tile * p.BN;
                if (!mbar_wait<EPI_BACKOFF_NS>(epi_done_bar(e), (e_phase >> e) & 1u, abort_flag)) {
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
                tma_store_wait_read();
                mbar_arrive(epi_free_bar(e));
                if (++e == p.nepi) e = 0;
            }
            tma_store_wait_read();
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

// ------------------------------------------------------------------------------------------------ CTA-pair variant
// For layers whose time is the L2 -> shared-memory traffic of the weight tiles (few output pixels against a large
// K x C x R x S weight tensor: the 14x14 and 7x7 stages of a ResNet at batch 64, deep 3x3 layers in general): two CTAs on
// neighbouring SMs (a cluster of two) compute one tile of 256 pixels x BN channels with tcgen05.mma.cta_group::2. Each
// CTA loads its own 128 rows of A and HALF of the B tile (BN/2 output channels), the MMA reads both halves across the
// pair, and each CTA finishes its own 128 rows from its own TMEM (bias, residual, activation, store) as in the plain
// kernel. Per k-block a CTA fetches 16 KB + BN x 64 B instead of 16 KB + BN x 128 B. Every load
// lands in the shared memory of the CTA that issued it.
// Protocol (even CTA = leader): `full` barriers live in the leader and count one arrive.expect_tx from each CTA's
// producer plus the bytes of both CTAs' loads; `empty` and `tfull` barriers are per CTA and are signalled by the
// leader's MMA thread with one commit per CTA; the leader's `tempty` barriers count the epilogue warps of both CTAs.
// Plain mode only (A by tiled or im2col TMA, B streamed per k-block, one 128-pixel sub-tile per CTA).
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_r, const __grid_constant__ CUtensorMap tmap_y,
                 const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_half_bytes = static_cast<uint32_t>(p.BN / 2) * BK * 2;     // this CTA's half of a weight k-block
    const uint32_t stage_bytes = A_STAGE_BYTES + b_half_bytes;
    const uint32_t epi_base = smem_base + static_cast<uint32_t>(p.stages) * stage_bytes;
    const uint32_t epi_bytes = static_cast<uint32_t>(p.nsub) * SUB_BYTES;
    const uint32_t bar_base = epi_base + static_cast<uint32_t>(p.nepi) * epi_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + MAX_ACC + a); };
    auto res_full_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + e); };
    auto epi_done_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + MAX_EPI + e); };
    auto epi_free_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + 2 * MAX_EPI + e); };
    const uint32_t misc_off = (bar_base - smem_u32(smem_raw)) + 8u * NUM_BARRIERS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + misc_off + 4);
    const uint32_t bias_off = misc_off + MISC_BYTES;
    const uint32_t bias_base = smem_u32(smem_raw) + bias_off;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: its peer
    const int pair = static_cast<int>(blockIdx.x >> 1), npairs = static_cast<int>(gridDim.x >> 1);
    const int total_tiles = p.m_tiles * p.n_tiles;    // m_tiles counts 256-pixel tiles here
    // Tile number `it` of this pair: pair, pair + npairs, ... with the n-tile fastest; this CTA's rows start at m0.
    auto tile_at2 = [&](int it, int& m0, int& n0) {
        const int tile = pair + it * npairs;
        if (tile >= total_tiles) return false;
        int m_tile = static_cast<int>(fastdiv(static_cast<uint32_t>(tile), p.div_ntiles));
        n0 = (tile - m_tile * p.n_tiles) * p.BN;
        if (p.rev) m_tile = p.m_tiles - 1 - m_tile;
        m0 = (2 * m_tile + static_cast<int>(rank)) * BM;
        return true;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 2);               // one arrive.expect_tx per CTA of the pair (used in the leader only)
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < p.nacc; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 2 * EPI_WARPS);  // the epilogue warps of both CTAs (used in the leader only)
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
        tmem_pair_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), static_cast<uint32_t>(p.tmem_cols));
        tmem_pair_relinquish();
    }
    // Both CTAs' barriers exist before either CTA signals one of the other's.
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int e = 0;
            uint32_t e_phase = 0;
            bool ok = true;
            const int PQ = p.P * p.Q;
            const uint32_t lead_full0 = mapa_shared(full_bar(0), 0);    // the leader's `full` barriers, 8 bytes apart
            const int b_row0 = static_cast<int>(rank) * (p.BN / 2);     // this CTA's half of the n-tile
            const unsigned long long pol_a = (p.hints & 1) ? l2_policy_evict_first() : 0ull;
            const unsigned long long pol_r = (p.hints & 2) ? l2_policy_evict_first() : 0ull;
            int m0, n0;
            // Weights are constants: the B halves of the first k-blocks (one per pipeline stage) are requested before the
            // wait for the preceding kernel, their barriers armed for the whole stage; the A tiles follow after the wait.
            int pre = 0;
            for (int pit = 0; pre < p.stages && tile_at2(pit, m0, n0); ++pit) {
                int tap = 0, cc = 0;
                for (int kb = 0; kb < p.kblocks && pre < p.stages; ++kb, ++pre) {
                    const uint32_t bar = lead_full0 + 8u * static_cast<uint32_t>(pre);
                    mbar_expect_tx_cluster(bar, stage_bytes);
                    tma_pair_load_3d(smem_base + static_cast<uint32_t>(pre) * stage_bytes + A_STAGE_BYTES, &tmap_b, bar, cc * BK,
                                     tap, n0 + b_row0);
                    if (++cc == p.cchunks) { cc = 0; ++tap; }
                }
            }
            int issued = 0;       // k-blocks issued so far (the first `pre` have their barrier armed and B on the way)
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int pit = 0; ok && tile_at2(pit, m0, n0); ++pit) {
                if (p.has_res) {
                    if (!mbar_wait(epi_free_bar(e), ((e_phase >> e) & 1u) ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    e_phase ^= 1u << e;
                    const int nsub = min(p.nsub, (p.K - n0 + 63) >> 6);
                    mbar_expect_tx(res_full_bar(e), static_cast<uint32_t>(nsub) * SUB_BYTES);
                    for (int sub = 0; sub < nsub; ++sub)      // rows past M: zero fill
                        tma_load_2d(epi_base + static_cast<uint32_t>(e) * epi_bytes + static_cast<uint32_t>(sub) * SUB_BYTES,
                                    &tmap_r, res_full_bar(e), n0 + sub * 64, m0, pol_r);
                    if (++e == p.nepi) e = 0;
                }
                // a peer whose 128 rows lie past the last pixel loads the leader's rows instead (its results are dropped)
                const int ml = m0 < p.M ? m0 : m0 - BM;
                int img = 0, h0 = 0, w0 = 0;
                if (p.im2col) {
                    img = static_cast<int>(fastdiv(static_cast<uint32_t>(ml), p.div_pq));
                    const int rem = ml - img * PQ;
                    const int pp = static_cast<int>(fastdiv(static_cast<uint32_t>(rem), p.div_q));
                    const int qq = rem - pp * p.Q;
                    h0 = pp * p.sh - p.ph;
                    w0 = qq * p.sw - p.pw;
                }
                int tap = 0, cc = 0, r = 0, s = 0;
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    const bool armed = issued < pre;      // this stage's barrier and B half were set up before the wait
                    ++issued;
                    if (!armed && !mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + static_cast<uint32_t>(stage) * stage_bytes;
                    const uint32_t bar = lead_full0 + 8u * static_cast<uint32_t>(stage);
                    if (!armed) {
                        mbar_expect_tx_cluster(bar, stage_bytes);
                        tma_pair_load_3d(a_dst + A_STAGE_BYTES, &tmap_b, bar, cc * BK, tap, n0 + b_row0);
                    }
                    if (p.im2col)
                        tma_pair_load_im2col_4d(a_dst, &tmap_a, bar, cc * BK, w0, h0, img,
                                                static_cast<uint16_t>(s * p.dw), static_cast<uint16_t>(r * p.dh), pol_a);
                    else
                        tma_pair_load_2d(a_dst, &tmap_a, bar, cc * BK, ml, pol_a);
                    if (++cc == p.cchunks) {
                        cc = 0;
                        ++tap;
                        if (++s == p.S) { s = 0; ++r; }
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (ok) {       // no bulk load of this CTA in flight, no MMA still reading its shared memory, when it exits
                for (int i = 0; i < p.stages; ++i) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) break;
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (rank == 0 && elect_one()) {
            const uint32_t idesc = umma_idesc_f16_f32(2 * BM, p.BN);
            const uint32_t hi128 = static_cast<uint32_t>(umma_desc_sw128(0) >> 32);
            auto lo_of = [](uint32_t addr) { return ((addr & 0x3ffffu) >> 4) | 0x10000u; };
            const uint32_t stage_step = stage_bytes >> 4;
            const uint32_t a_lo0 = lo_of(smem_base);
            const uint32_t peer_empty0 = mapa_shared(empty_bar(0), 1);
            const uint32_t peer_tfull0 = mapa_shared(tfull_bar(0), 1);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t st_lo = a_lo0;
            uint32_t acc_phase = 0;
            int acc = -1;
            bool failed = false;
            uint32_t st_ready = 0;
            int m0, n0;
            for (int it = 0; tile_at2(it, m0, n0); ++it) {
                if (++acc == p.nacc) acc = 0;
                failed |= !mbar_wait(tempty_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag);
                acc_phase ^= 1u << acc;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.acc_stride);
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!st_ready) failed |= !mbar_wait(full_bar(stage), phase, abort_flag);
                    tc_fence_after();
                    {
                        const bool wrap = stage + 1 == p.stages;
                        st_ready = mbar_test(full_bar(wrap ? 0 : stage + 1), wrap ? phase ^ 1u : phase);
                    }
                    umma_pair_f16_kblock(d_tmem, st_lo, hi128, st_lo + (A_STAGE_BYTES >> 4), hi128, idesc,
                                         static_cast<uint32_t>(kb != 0));
                    umma_pair_commit(empty_bar(stage));                                      // frees the stage in both CTAs
                    umma_pair_commit(peer_empty0 + 8u * static_cast<uint32_t>(stage));
                    st_lo += stage_step;
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; st_lo = a_lo0; }
                }
                umma_pair_commit(tfull_bar(acc));                                            // both halves of the accumulator
                umma_pair_commit(peer_tfull0 + 8u * static_cast<uint32_t>(acc));
            }
            if (failed) atomicExch(p.status, STATUS_WAIT_MMA);
        }
        __syncwarp();
    } else if (warp < STORE_WARP) {
        // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int lane_group = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row = lane_group * 32 + lane;
        const uint32_t row_xor = static_cast<uint32_t>(row & 7);
        const uint32_t bias_s = bias_base;
        const uint32_t stage0 = epi_base + static_cast<uint32_t>(row) * 128u;
        {
            float* bias_f = reinterpret_cast<float*>(smem_raw + bias_off);
            for (int i = threadIdx.x - 64; i < p.bias_elems; i += EPI_WARPS * 32)
                bias_f[i] = (p.bias != nullptr && i < p.K) ? __half2float(p.bias[i]) : 0.f;
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        }
        const uint32_t lead_tempty0 = mapa_shared(tempty_bar(0), 0);
        uint32_t acc_phase = 0, e_phase = 0;
        int e = 0, acc = -1;
        bool ok = true;
        const int act_t = (p.act == 0 || p.act == 1 || p.act == 3 || p.act == 5) ? p.act : 2;
        const int variant = act_t * 2 + (p.has_res ? 1 : 0);
        int m0, n0;
        for (int it = 0; ok && tile_at2(it, m0, n0); ++it) {
            if (++acc == p.nacc) acc = 0;
            const bool got_buf = p.has_res ? mbar_wait<EPI_BACKOFF_NS>(res_full_bar(e), (e_phase >> e) & 1u, abort_flag)
                                           : mbar_wait<EPI_BACKOFF_NS>(epi_free_bar(e), ((e_phase >> e) & 1u) ^ 1u, abort_flag);
            if (!got_buf || !mbar_wait<EPI_BACKOFF_NS>(tfull_bar(acc), (acc_phase >> acc) & 1u, abort_flag)) {
                if (lane == 0) atomicExch(p.status, STATUS_WAIT_EPILOGUE);
                ok = false;
                break;
            }
            e_phase ^= 1u << e;
            acc_phase ^= 1u << acc;
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                                   static_cast<uint32_t>(acc * p.acc_stride);
            const uint32_t stage_row0 = stage0 + static_cast<uint32_t>(e) * epi_bytes;
            const int ncols = min(p.BN, p.K - n0);
            switch (variant) {
                case 0: epilogue_rows<0, false>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 1: epilogue_rows<0, true>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 2: epilogue_rows<1, false>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 3: epilogue_rows<1, true>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 4: epilogue_rows<2, false>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 5: epilogue_rows<2, true>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 6: epilogue_rows<3, false>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 7: epilogue_rows<3, true>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                case 10: epilogue_rows<5, false>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
                default: epilogue_rows<5, true>(p, t_row, stage_row0, row_xor, bias_s, n0, ncols, group); break;
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(lead_tempty0 + 8u * static_cast<uint32_t>(acc));   // this CTA's half may be overwritten
                mbar_arrive(epi_done_bar(e));
            }
            if (++e == p.nepi) e = 0;
        }
    } else {
        // ------------------------------------------------------------------ store warp (both CTAs)
        if (elect_one()) {
            uint32_t e_phase = 0;
            int e = 0;
            const unsigned long long pol_y = (p.hints & 4) ? l2_policy_evict_last() : 0ull;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            int m0, n0;
            for (int sit = 0; ok && tile_at2(sit, m0, n0); ++sit) {
                if (!mbar_wait<EPI_BACKOFF_NS>(epi_done_bar(e), (e_phase >> e) & 1u, abort_flag)) {
                    atomicExch(p.status, STATUS_WAIT_STORE);
                    ok = false;
                    break;
                }
                e_phase ^= 1u << e;
                const int nsub = min(p.nsub, (p.K - n0 + 63) >> 6);
                if (m0 < p.M) {
                    for (int sub = 0; sub < nsub; ++sub)
                        tma_store_2d(&tmap_y, epi_base + static_cast<uint32_t>(e) * epi_bytes + static_cast<uint32_t>(sub) * SUB_BYTES,
                                     n0 + sub * 64, m0, pol_y);
                    tma_store_commit();
                    tma_store_wait_read();
                }
                mbar_arrive(epi_free_bar(e));
                if (++e == p.nepi) e = 0;
            }
            tma_store_wait_read();
        }
    }

    // Neither CTA leaves (or frees TMEM) while the other may still signal its barriers or read its shared memory.
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_pair_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
    }
}

// ------------------------------------------------------------------------------------------------ layer chains
// A run of consecutive convolutions (the bottleneck blocks of a ResNet stage, say) as ONE launch of CTA pairs: the
// tiles of all layers form one sequence (layer by layer, 256 pixels x BN channels each, as in conv_pair_kernel), pair
// i takes tiles i, i + pairs, i + 2 pairs, ..., and a tile starts as soon as the tiles of earlier layers that hold its
// input pixels (and its residual tile) are complete. What this removes against one launch per layer: the launch /
// set-up / drain latency between layers (about 3.5 us each), the idle SMs of every layer's last partial wave (the next
// layer's first tiles run there), and the cold start of each layer's pipeline (weights of the next tile are requested
// while the dependency is still being waited for).
// Completion is tracked per layer and 256-row tile by a counter in global memory: the store thread of each of the
// tile's 2 * n_tiles CTA-tiles adds one after its bulk stores have completed (cp.async.bulk.wait_group 0, proxy fence,
// release at GPU scope); a producer thread that needs rows [lo, hi] of an earlier layer's output polls (bounded) the
// counters of the tiles that hold them (acquire at GPU scope, then a proxy fence before its bulk loads). Every pair
// walks its tiles in increasing order and a tile depends on tiles of earlier layers only, so the pair that holds the
// lowest unfinished tile can always proceed: no deadlock as long as all pairs are resident, which the grid size
// (at most the number of clusters the device runs at once) guarantees. The host zeroes the counters before the launch
// and makes sure no buffer of the chain aliases another (layers no longer run in stream order).
// Shared-memory map: [stages x slot (A 16 KB | B half up to maxBN x 64 B)] [staging region, cut per layer into
// buffers of nsub x 16 KB] [barriers] [tmem slot, abort flag, released-tile counter] [bias copy of the current layer].
// A staging buffer is free once the store thread has counted the tile that used it last; where consecutive layers
// cut the region differently (tiles of another width) the first tile of the new cut waits for all earlier tiles.
static constexpr int CHAIN_MAX_LAYERS = 48;
static constexpr int CHAIN_MAX_EXT_RES = 4;
static constexpr int STATUS_WAIT_CHAIN = 0x108;

struct ChainLayer {
    CUtensorMap tmap_a, tmap_b, tmap_y;   // the residual of a layer is read through the output map of layer res_layer
    const __half* bias;
    const float* scale;
    int M, K, P, Q, H, W, S;       // output rows / channels / map, input map, filter width
    int sh, sw, ph, pw, dh, dw, rspan;   // rspan = (R - 1) * dh
    int cchunks, kblocks, BN, n_tiles, m_tiles, nsub, nepi, im2col, act, has_res;
    int tile0;                     // index of the layer's first tile in the chain's tile sequence
    int in_layer, res_layer;       // layers of the chain that produce this layer's input / residual (-1: from outside)
    int res_ext;                   // residual from outside the chain: index into ChainParams::ext_res
    int flag0;                     // index of the layer's first completion counter (one per 256-row tile)
    int done_count;                // 2 * n_tiles: arrivals that complete one 256-row tile
    int bias_elems;
    FastDiv div_ntiles, div_pq, div_q;
};
struct ChainParams {
    int n_layers, total_tiles, stages;
    uint32_t stage_bytes, epi_region_bytes;
    int* flags;
    int* status;
    CUtensorMap ext_res[CHAIN_MAX_EXT_RES];   // residuals that no layer of the chain produces
    ChainLayer L[CHAIN_MAX_LAYERS];
};
static_assert(sizeof(ChainParams) <= 32 * 1024 - 256, "kernel parameters are limited to 32764 bytes");

// Bounded wait until *flag >= need. Returns false (and raises the CTA's abort flag) when it gives up.
__device__ __forceinline__ bool chain_wait_flag(const int* flag, int need, volatile int* abort_flag) {
    if (ld_acquire_gpu(flag) >= need) return true;
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    for (;;) {
        __nanosleep(32);
        if (ld_acquire_gpu(flag) >= need) return true;
        if ((++spins & 0x3f) == 0) {
            if (*abort_flag) return false;
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
        }
    }
}

__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_chain_kernel(const __grid_constant__ ChainParams cp) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t stage_bytes = cp.stage_bytes;
    const uint32_t epi_base = smem_base + static_cast<uint32_t>(cp.stages) * stage_bytes;
    const uint32_t bar_base = epi_base + cp.epi_region_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + MAX_ACC + a); };
    auto res_full_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + e); };
    auto epi_done_bar = [&](int e) { return bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + MAX_EPI + e); };
    const uint32_t epi_sync_bar = bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC + 3 * MAX_EPI);   // the epilogue warps among themselves
    const uint32_t misc_off = (bar_base - smem_u32(smem_raw)) + 8u * NUM_BARRIERS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + misc_off + 4);
    // number of this CTA's tiles whose staging buffer the store thread has released. A role that starts a layer whose
    // staging buffers are cut differently waits until every earlier tile is counted here: barrier parities cannot say
    // that, a role that did not take the buffers itself may be several uses ahead of their release.
    volatile int* released = reinterpret_cast<volatile int*>(smem_raw + misc_off + 8);
    static_assert(MISC_BYTES >= 12, "tmem slot, abort flag, released-tile counter");
    const uint32_t bias_off = misc_off + MISC_BYTES;
    const uint32_t bias_base = smem_u32(smem_raw) + bias_off;
    constexpr int NACC = 2;
    constexpr uint32_t ACC_STRIDE = 256;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = static_cast<int>(blockIdx.x >> 1), npairs = static_cast<int>(gridDim.x >> 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < cp.stages; ++s) {
            mbar_init(full_bar(s), 2);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < NACC; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 2 * EPI_WARPS);
        }
        for (int e = 0; e < MAX_EPI; ++e) {
            mbar_init(res_full_bar(e), 1);
            mbar_init(epi_done_bar(e), EPI_WARPS);
        }
        mbar_init(epi_sync_bar, EPI_WARPS);
        *abort_flag = 0;
        *released = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_pair_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), NACC * ACC_STRIDE);
        tmem_pair_relinquish();
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Layer of tile g, given the layer of the previous (lower) tile of this thread.
    auto advance = [&](int g, int l) {
        while (l + 1 < cp.n_layers && g >= cp.L[l + 1].tile0) ++l;
        return l;
    };

    // Bounded wait until the store thread has released the staging buffers of this CTA's first `need` tiles.
    auto wait_released = [&](int need) {
        unsigned long long t0 = 0;
        uint32_t spins = 0;
        while (*released < need) {
            __nanosleep(32);
            if ((++spins & 0x3f) == 0) {
                if (*abort_flag) return false;
                const unsigned long long now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
            }
        }
        __threadfence_block();
        return true;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int e = 0;
            bool ok = true;
            const uint32_t lead_full0 = mapa_shared(full_bar(0), 0);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int l = -1;
            int it = 0;               // tiles of this CTA before the current one
            int cut = 0, it0 = 0;     // how the staging region is cut (sub-tiles per buffer) and since which tile
            for (int g = pair; ok && g < cp.total_tiles; g += npairs, ++it) {
                const int nl = advance(g, l < 0 ? 0 : l);
                const bool switched = nl != l;
                l = nl;
                const ChainLayer& L = cp.L[l];
                if (switched) {
                    tma_prefetch_desc(&L.tmap_a);
                    tma_prefetch_desc(&L.tmap_b);
                    if (L.nsub != cut) { cut = L.nsub; e = 0; it0 = it; }
                }
                const int t = g - L.tile0;
                const int m_tile = static_cast<int>(fastdiv(static_cast<uint32_t>(t), L.div_ntiles));
                const int n0 = (t - m_tile * L.n_tiles) * L.BN;
                const int m0 = (2 * m_tile + static_cast<int>(rank)) * BM;
                const uint32_t b_half_bytes = static_cast<uint32_t>(L.BN / 2) * BK * 2;
                const uint32_t tx_bytes = A_STAGE_BYTES + b_half_bytes;
                const uint32_t epi_bytes = static_cast<uint32_t>(L.nsub) * SUB_BYTES;
                if (L.has_res) {
                    // staging buffer e: free once the tile that used it last (nepi tiles ago) has been stored; after a
                    // change of the cut, once every earlier tile has been
                    if (!wait_released(max(it0, it - L.nepi + 1))) {
                        atomicExch(cp.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    if (L.res_layer >= 0) {
                        const ChainLayer& R = cp.L[L.res_layer];
                        if (!chain_wait_flag(cp.flags + R.flag0 + m_tile, R.done_count, abort_flag)) {
                            atomicExch(cp.status, STATUS_WAIT_CHAIN);
                            ok = false;
                            break;
                        }
                        asm volatile("fence.proxy.async;" ::: "memory");
                    }
                    const CUtensorMap* rmap = L.res_layer >= 0 ? &cp.L[L.res_layer].tmap_y : &cp.ext_res[L.res_ext];
                    const int nsub = min(L.nsub, (L.K - n0 + 63) >> 6);
                    mbar_expect_tx(res_full_bar(e), static_cast<uint32_t>(nsub) * SUB_BYTES);
                    for (int sub = 0; sub < nsub; ++sub)
                        tma_load_2d(epi_base + static_cast<uint32_t>(e) * epi_bytes + static_cast<uint32_t>(sub) * SUB_BYTES,
                                    rmap, res_full_bar(e), n0 + sub * 64, m0);
                }
                if (++e == L.nepi) e = 0;

                const int ml = m0 < L.M ? m0 : m0 - BM;     // a peer without rows loads the leader's (results dropped)
                const int PQ = L.P * L.Q;
                int img = 0, pp = 0, h0 = 0, w0 = 0;
                {
                    img = static_cast<int>(fastdiv(static_cast<uint32_t>(ml), L.div_pq));
                    const int rem = ml - img * PQ;
                    pp = static_cast<int>(fastdiv(static_cast<uint32_t>(rem), L.div_q));
                    const int qq = rem - pp * L.Q;
                    h0 = pp * L.sh - L.ph;
                    w0 = qq * L.sw - L.pw;
                }
                const int b_row0 = n0 + static_cast<int>(rank) * (L.BN / 2);
                int tap = 0, cc = 0, r = 0, s = 0;
                for (int kb = 0; kb < L.kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicExch(cp.status, STATUS_WAIT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + static_cast<uint32_t>(stage) * stage_bytes;
                    const uint32_t bar = lead_full0 + 8u * static_cast<uint32_t>(stage);
                    mbar_expect_tx_cluster(bar, tx_bytes);
                    tma_pair_load_3d(a_dst + A_STAGE_BYTES, &L.tmap_b, bar, cc * BK, tap, b_row0);    // weights: no dependency
                    if (kb == 0 && L.in_layer >= 0) {
                        // input pixels of this CTA's rows [ml, last]: from the first needed input row of the first image to
                        // the last needed input row of the last image, as rows of the producing layer's output
                        const ChainLayer& I = cp.L[L.in_layer];
                        const int last = min(ml + BM, L.M) - 1;
                        const int img1 = static_cast<int>(fastdiv(static_cast<uint32_t>(last), L.div_pq));
                        const int pp1 = static_cast<int>(fastdiv(static_cast<uint32_t>(last - img1 * PQ), L.div_q));
                        const int HW = L.H * L.W;
                        const int lo = img * HW + max(0, pp * L.sh - L.ph) * L.W;
                        const int hi = img1 * HW + min(L.H - 1, pp1 * L.sh - L.ph + L.rspan) * L.W + L.W - 1;
                        bool seen = true;
                        for (int f = lo >> 8; seen && f <= (hi >> 8); ++f)
                            seen = chain_wait_flag(cp.flags + I.flag0 + f, I.done_count, abort_flag);
                        if (!seen) {
                            atomicExch(cp.status, STATUS_WAIT_CHAIN);
                            ok = false;
                            break;
                        }
                        asm volatile("fence.proxy.async;" ::: "memory");
                    }
                    if (L.im2col)
                        tma_pair_load_im2col_4d(a_dst, &L.tmap_a, bar, cc * BK, w0, h0, img,
                                                static_cast<uint16_t>(s * L.dw), static_cast<uint16_t>(r * L.dh));
                    else
                        tma_pair_load_2d(a_dst, &L.tmap_a, bar, cc * BK, ml);
                    if (++cc == L.cchunks) {
                        cc = 0;
                        ++tap;
                        if (++s == L.S) { s = 0; ++r; }
                    }
                    if (++stage == cp.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (ok) {
                for (int i = 0; i < cp.stages; ++i) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) break;
                    if (++stage == cp.stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (rank == 0 && elect_one()) {
            const uint32_t hi128 = static_cast<uint32_t>(umma_desc_sw128(0) >> 32);
            auto lo_of = [](uint32_t addr) { return ((addr & 0x3ffffu) >> 4) | 0x10000u; };
            const uint32_t stage_step = stage_bytes >> 4;
            const uint32_t a_lo0 = lo_of(smem_base);
            const uint32_t peer_empty0 = mapa_shared(empty_bar(0), 1);
            const uint32_t peer_tfull0 = mapa_shared(tfull_bar(0), 1);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t st_lo = a_lo0;
            uint32_t acc_phase = 0;
            int acc = -1;
            bool failed = false;
            uint32_t st_ready = 0;
            int l = 0;
            for (int g = pair; g < cp.total_tiles; g += npairs) {
                l = advance(g, l);
                const int kblocks = cp.L[l].kblocks;
                const uint32_t idesc = umma_idesc_f16_f32(2 * BM, cp.L[l].BN);
                if (++acc == NACC) acc = 0;
                failed |= !mbar_wait(tempty_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag);
                acc_phase ^= 1u << acc;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * ACC_STRIDE;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!st_ready) failed |= !mbar_wait(full_bar(stage), phase, abort_flag);
                    tc_fence_after();
                    {
                        const bool wrap = stage + 1 == cp.stages;
                        st_ready = mbar_test(full_bar(wrap ? 0 : stage + 1), wrap ? phase ^ 1u : phase);
                    }
                    umma_pair_f16_kblock(d_tmem, st_lo, hi128, st_lo + (A_STAGE_BYTES >> 4), hi128, idesc,
                                         static_cast<uint32_t>(kb != 0));
                    umma_pair_commit(empty_bar(stage));
                    umma_pair_commit(peer_empty0 + 8u * static_cast<uint32_t>(stage));
                    st_lo += stage_step;
                    if (++stage == cp.stages) { stage = 0; phase ^= 1u; st_lo = a_lo0; }
                }
                umma_pair_commit(tfull_bar(acc));
                umma_pair_commit(peer_tfull0 + 8u * static_cast<uint32_t>(acc));
            }
            if (failed) atomicExch(cp.status, STATUS_WAIT_MMA);
        }
        __syncwarp();
    } else if (warp < STORE_WARP) {
        // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int lane_group = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row = lane_group * 32 + lane;
        const uint32_t row_xor = static_cast<uint32_t>(row & 7);
        const uint32_t stage0 = epi_base + static_cast<uint32_t>(row) * 128u;
        float* bias_f = reinterpret_cast<float*>(smem_raw + bias_off);
        const uint32_t lead_tempty0 = mapa_shared(tempty_bar(0), 0);
        uint32_t acc_phase = 0, r_phase = 0, sync_phase = 0;
        int e = 0, acc = -1;
        bool ok = true;
        int l = -1;
        int it = 0, cut = 0, it0 = 0;
        // All epilogue warps meet (a bounded wait on an mbarrier, not bar.sync: a warp that has given up never arrives).
        auto epi_sync = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_sync_bar);
            const bool met = mbar_wait<EPI_BACKOFF_NS>(epi_sync_bar, sync_phase, abort_flag);
            sync_phase ^= 1u;
            return met;
        };
        ConvParams ep;       // the epilogue code reads the activation code and the scale pointer from here
        ep.act = 0;
        ep.scale = nullptr;
        int variant = 0;
        for (int g = pair; ok && g < cp.total_tiles; g += npairs, ++it) {
            const int nl = advance(g, l < 0 ? 0 : l);
            const bool switched = nl != l;
            l = nl;
            const ChainLayer& L = cp.L[l];
            if (switched) {
                // every epilogue warp is past the previous layer's last tile before its bias copy is replaced
                ok = epi_sync();
                for (int i = threadIdx.x - 64; i < L.bias_elems; i += EPI_WARPS * 32)
                    bias_f[i] = (L.bias != nullptr && i < L.K) ? __half2float(L.bias[i]) : 0.f;
                ok = epi_sync() && ok;
                ep.act = L.act;
                ep.scale = L.scale;
                const int act_t = (L.act == 0 || L.act == 1 || L.act == 3 || L.act == 5) ? L.act : 2;
                variant = act_t * 2 + (L.has_res ? 1 : 0);
                if (L.nsub != cut) { cut = L.nsub; e = 0; it0 = it; }
            }
            const int t = g - L.tile0;
            const int m_tile = static_cast<int>(fastdiv(static_cast<uint32_t>(t), L.div_ntiles));
            const int n0 = (t - m_tile * L.n_tiles) * L.BN;
            const uint32_t epi_bytes = static_cast<uint32_t>(L.nsub) * SUB_BYTES;
            if (++acc == NACC) acc = 0;
            bool got_buf = ok;
            if (got_buf) {
                if (L.has_res) {
                    got_buf = mbar_wait<EPI_BACKOFF_NS>(res_full_bar(e), (r_phase >> e) & 1u, abort_flag);
                    r_phase ^= 1u << e;
                } else {
                    got_buf = wait_released(max(it0, it - L.nepi + 1));
                }
            }
            if (!got_buf || !mbar_wait<EPI_BACKOFF_NS>(tfull_bar(acc), (acc_phase >> acc) & 1u, abort_flag)) {
                if (lane == 0) atomicExch(cp.status, STATUS_WAIT_EPILOGUE);
                ok = false;
                break;
            }
            acc_phase ^= 1u << acc;
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + static_cast<uint32_t>(acc) * ACC_STRIDE;
            const uint32_t stage_row0 = stage0 + static_cast<uint32_t>(e) * epi_bytes;
            const int ncols = min(L.BN, L.K - n0);
            // epilogue_rows lays a tile's 64-channel sub-tiles SUB_BYTES apart, as this layer's staging buffers are
            switch (variant) {
                case 0: epilogue_rows<0, false>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 1: epilogue_rows<0, true>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 2: epilogue_rows<1, false>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 3: epilogue_rows<1, true>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 4: epilogue_rows<2, false>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 5: epilogue_rows<2, true>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 6: epilogue_rows<3, false>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 7: epilogue_rows<3, true>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                case 10: epilogue_rows<5, false>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
                default: epilogue_rows<5, true>(ep, t_row, stage_row0, row_xor, bias_base, n0, ncols, group); break;
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(lead_tempty0 + 8u * static_cast<uint32_t>(acc));
                mbar_arrive(epi_done_bar(e));
            }
            if (++e == L.nepi) e = 0;
        }
    } else {
        // ------------------------------------------------------------------ store warp (both CTAs)
        if (elect_one()) {
            uint32_t d_phase = 0;
            int e = 0;
            int n_released = 0;
            int cut = 0;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            int l = -1;
            for (int g = pair; ok && g < cp.total_tiles; g += npairs) {
                const int nl = advance(g, l < 0 ? 0 : l);
                if (nl != l) {
                    l = nl;
                    if (cp.L[l].nsub != cut) { cut = cp.L[l].nsub; e = 0; }
                    tma_prefetch_desc(&cp.L[l].tmap_y);
                }
                const ChainLayer& L = cp.L[l];
                const int t = g - L.tile0;
                const int m_tile = static_cast<int>(fastdiv(static_cast<uint32_t>(t), L.div_ntiles));
                const int n0 = (t - m_tile * L.n_tiles) * L.BN;
                const int m0 = (2 * m_tile + static_cast<int>(rank)) * BM;
                const uint32_t epi_bytes = static_cast<uint32_t>(L.nsub) * SUB_BYTES;
                if (!mbar_wait<EPI_BACKOFF_NS>(epi_done_bar(e), (d_phase >> e) & 1u, abort_flag)) {
                    atomicExch(cp.status, STATUS_WAIT_STORE);
                    ok = false;
                    break;
                }
                d_phase ^= 1u << e;
                if (m0 < L.M) {
                    const int nsub = min(L.nsub, (L.K - n0 + 63) >> 6);
                    for (int sub = 0; sub < nsub; ++sub)
                        tma_store_2d(&L.tmap_y, epi_base + static_cast<uint32_t>(e) * epi_bytes + static_cast<uint32_t>(sub) * SUB_BYTES,
                                     n0 + sub * 64, m0);
                    tma_store_commit();
                    tma_store_wait_read();
                }
                __threadfence_block();
                *released = ++n_released;      // the staging buffer may be refilled
                // this CTA's part of the tile is in global memory: count it for the layers that read it
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                asm volatile("fence.proxy.async;" ::: "memory");
                asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(cp.flags + L.flag0 + m_tile) : "memory");
                if (++e == L.nepi) e = 0;
            }
        }
    }

    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_pair_dealloc(tmem_base, NACC * ACC_STRIDE);
    }
}

// ------------------------------------------------------------------------------------------------ two layers, one launch
// z = act2(conv1x1(y, w2) + b2) with y = act1(conv1x1(x, w1) + b1 [+ res]): the last convolution of a bottleneck block
// (64 -> 256 channels, + identity, ReLU) and the first of the next block (256 -> 64), where the 256-channel map is by
// far the largest tensor of either layer. Each CTA walks 128-pixel tiles; a tile's y is produced in units of 128
// channels (z up to 64 channels wide; a unit = two 64-channel panels in the 128-byte-swizzled layout that TMA and the
// MMA unit share, ring of three slots) or of 64 channels (z up to 128 wide: one panel, ring of four):
//   GEMM 1 (A = x tile by TMA, B = w1 resident)  -> TMEM unit accumulator (one per slot)
//   epilogue 1: + bias (+ residual, which TMA put into the y slot) -> act1 -> fp16, in place in the y slot
//   the finished y slot is (a) stored to global memory by TMA and (b) read as the A operand of GEMM 2 (B = w2 resident),
//   one k-block per panel -> second accumulator (two buffers of 64 or 128 columns); the slot is free when both are done
//   epilogue 2: + bias -> act2 -> fp16 -> z staging panels -> TMA store.
// y is written once and never read back: the second layer costs its weights and its (small) output only. Results are
// those of two separate launches bit for bit: same fp16 y values, same order of the fp32 accumulation over K.
// Roles as in conv_tcgen05_kernel (producer lane, MMA lane, 16 epilogue warps, store lane); every wait is bounded.
static constexpr int DUAL_MAX_YSLOTS = 4;             // y unit slots = unit accumulators in TMEM (3 or 4 are used)
static constexpr int DUAL_MAX_SA = 4;                 // x-tile stages
static constexpr int DUAL_LAG = 2;                    // GEMM 2 of a unit is issued this many units behind GEMM 1
static constexpr int DUAL_NUM_BARRIERS = 1 + 2 * DUAL_MAX_SA + 5 * DUAL_MAX_YSLOTS + 4 + 2;
static constexpr int DUAL_MISC_BYTES = 16 + (DUAL_NUM_BARRIERS & 1) * 8;
static constexpr int STATUS_WAIT_DUAL = 0x109;

struct DualParams {
    int M, m_tiles;
    int kb1;            // input channels of the first layer / 64 (1 or 2)
    int K1, H;          // channels of y (128 or 256) and units per tile (K1 / UW)
    int UW, UP, ys;     // channels per unit (128 or 64), panels per unit (UW / 64), y slots (3 or 4; ys * UW <= 384)
    int N2;             // channels of z (multiple of 16, at most 128)
    int acc2_col, acc2_stride;   // TMEM column of the second accumulator's first buffer, columns between its two buffers
    int zp;             // 64-channel panels of the z staging tile (1 or 2)
    int act1, act2, has_res;
    int hints;          // bit 0: x is dead after this launch, bit 1: the residual is, bit 2: keep y in L2, bit 3: keep z
    int sa;             // x-tile stages
    const __half* bias1;
    const __half* bias2;
    int* status;
};

__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_dual_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w1,
                 const __grid_constant__ CUtensorMap tmap_r, const __grid_constant__ CUtensorMap tmap_y,
                 const __grid_constant__ CUtensorMap tmap_w2, const __grid_constant__ CUtensorMap tmap_z,
                 const DualParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t w1_kb_bytes = static_cast<uint32_t>(p.K1) * 128u;            // [K1][64] of one k-block
    const uint32_t w1_bytes = static_cast<uint32_t>(p.kb1) * w1_kb_bytes;
    const uint32_t w2_kb_bytes = static_cast<uint32_t>(p.N2) * 128u;            // [N2][64] of one k-block of GEMM 2
    const int kb2 = p.K1 >> 6;
    const uint32_t w2_bytes = static_cast<uint32_t>(kb2) * w2_kb_bytes;
    const uint32_t a_stage_bytes = static_cast<uint32_t>(p.kb1) * A_STAGE_BYTES;
    const uint32_t w1_base = smem_base;
    const uint32_t w2_base = w1_base + w1_bytes;
    const uint32_t a_base = w2_base + w2_bytes;
    const uint32_t y_base = a_base + static_cast<uint32_t>(p.sa) * a_stage_bytes;
    const uint32_t y_slot_bytes = static_cast<uint32_t>(p.UP) * SUB_BYTES;
    const uint32_t z_base = y_base + static_cast<uint32_t>(p.ys) * y_slot_bytes;
    const uint32_t bar_base = z_base + static_cast<uint32_t>(p.zp) * SUB_BYTES;
    const uint32_t w_full_bar = bar_base;
    auto a_full_bar = [&](int s) { return bar_base + 8u * (1 + s); };
    auto a_empty_bar = [&](int s) { return bar_base + 8u * (1 + DUAL_MAX_SA + s); };
    auto res_full_bar = [&](int s) { return bar_base + 8u * (1 + 2 * DUAL_MAX_SA + s); };
    auto acc1_full_bar = [&](int s) { return bar_base + 8u * (1 + 2 * DUAL_MAX_SA + DUAL_MAX_YSLOTS + s); };
    auto acc1_empty_bar = [&](int s) { return bar_base + 8u * (1 + 2 * DUAL_MAX_SA + 2 * DUAL_MAX_YSLOTS + s); };
    auto y_done_bar = [&](int s) { return bar_base + 8u * (1 + 2 * DUAL_MAX_SA + 3 * DUAL_MAX_YSLOTS + s); };
    auto y_free_bar = [&](int s) { return bar_base + 8u * (1 + 2 * DUAL_MAX_SA + 4 * DUAL_MAX_YSLOTS + s); };
    auto acc2_full_bar = [&](int b) { return bar_base + 8u * (1 + 2 * DUAL_MAX_SA + 5 * DUAL_MAX_YSLOTS + b); };
    auto acc2_empty_bar = [&](int b) { return bar_base + 8u * (1 + 2 * DUAL_MAX_SA + 5 * DUAL_MAX_YSLOTS + 2 + b); };
    const uint32_t z_done_bar = bar_base + 8u * (1 + 2 * DUAL_MAX_SA + 5 * DUAL_MAX_YSLOTS + 4);
    const uint32_t z_free_bar = z_done_bar + 8u;
    const uint32_t misc_off = (bar_base - smem_u32(smem_raw)) + 8u * DUAL_NUM_BARRIERS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + misc_off + 4);
    static_assert((8 * DUAL_NUM_BARRIERS + DUAL_MISC_BYTES) % 16 == 0, "bias copies must be 16-byte aligned");
    const uint32_t bias_off = misc_off + DUAL_MISC_BYTES;
    const uint32_t bias1_s = smem_u32(smem_raw) + bias_off;                    // fp32 [K1], then fp32 [N2]
    const uint32_t bias2_s = bias1_s + 4u * static_cast<uint32_t>(p.K1);

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int T = static_cast<int>(blockIdx.x) < p.m_tiles
                      ? (p.m_tiles - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;   // tiles of this CTA
    const int U = T * p.H;                                                                                       // halves
    auto tile_row0 = [&](int it) { return (static_cast<int>(blockIdx.x) + it * static_cast<int>(gridDim.x)) * BM; };

    if (threadIdx.x == 0) {
        mbar_init(w_full_bar, 1);
        for (int s = 0; s < p.sa; ++s) {
            mbar_init(a_full_bar(s), 1);
            mbar_init(a_empty_bar(s), 1);
        }
        for (int s = 0; s < p.ys; ++s) {
            mbar_init(res_full_bar(s), 1);
            mbar_init(acc1_full_bar(s), 1);
            mbar_init(acc1_empty_bar(s), EPI_WARPS);
            mbar_init(y_done_bar(s), EPI_WARPS);
            mbar_init(y_free_bar(s), 2);            // the store has read the slot out + GEMM 2 has read it
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc2_full_bar(b), 1);
            mbar_init(acc2_empty_bar(b), EPI_WARPS);
        }
        mbar_init(z_done_bar, EPI_WARPS);
        mbar_init(z_free_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_w1);
        tma_prefetch_desc(&tmap_w2);
        tma_prefetch_desc(&tmap_y);
        tma_prefetch_desc(&tmap_z);
        if (p.has_res) tma_prefetch_desc(&tmap_r);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512u);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            const unsigned long long pol_a = (p.hints & 1) ? l2_policy_evict_first() : 0ull;
            const unsigned long long pol_r = (p.hints & 2) ? l2_policy_evict_first() : 0ull;
            if (T > 0) {      // both weight tensors, once (constants: fetched before the dependency wait)
                mbar_expect_tx(w_full_bar, w1_bytes + w2_bytes);
                for (int kb = 0; kb < p.kb1; ++kb)
                    for (int r = 0; r < p.K1; r += 128)      // boxes of 128 rows, row r of a k-block at r * 128 bytes
                        tma_load_3d(w1_base + static_cast<uint32_t>(kb) * w1_kb_bytes + static_cast<uint32_t>(r) * 128u,
                                    &tmap_w1, w_full_bar, kb * BK, 0, r);
                for (int kb = 0; kb < kb2; ++kb)
                    tma_load_3d(w2_base + static_cast<uint32_t>(kb) * w2_kb_bytes, &tmap_w2, w_full_bar, kb * BK, 0, 0);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            int u = 0;
            for (int it = 0; ok && it < T; ++it) {
                const int m0 = tile_row0(it);
                const int sa = it % p.sa;
                if (!mbar_wait(a_empty_bar(sa), (static_cast<uint32_t>(it / p.sa) & 1u) ^ 1u, abort_flag)) {
                    atomicExch(p.status, STATUS_WAIT_DUAL);
                    break;
                }
                mbar_expect_tx(a_full_bar(sa), a_stage_bytes);
                for (int kb = 0; kb < p.kb1; ++kb)
                    tma_load_2d(a_base + static_cast<uint32_t>(sa) * a_stage_bytes + static_cast<uint32_t>(kb) * A_STAGE_BYTES, &tmap_a,
                                a_full_bar(sa), kb * BK, m0, pol_a);
                if (!p.has_res) continue;
                for (int h = 0; h < p.H; ++h, ++u) {
                    const int s = u % p.ys;
                    if (!mbar_wait(y_free_bar(s), (static_cast<uint32_t>(u / p.ys) & 1u) ^ 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_DUAL);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(res_full_bar(s), y_slot_bytes);
                    for (int j = 0; j < p.UP; ++j)
                        tma_load_2d(y_base + static_cast<uint32_t>(s) * y_slot_bytes + static_cast<uint32_t>(j) * SUB_BYTES, &tmap_r,
                                    res_full_bar(s), h * p.UW + j * 64, m0, pol_r);
                }
            }
            // no bulk load of this CTA may be in flight when it exits: x tiles are consumed by GEMM 1 and residual
            // halves by epilogue 1, both of which the closing barrier waits for
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            const uint32_t idesc1 = umma_idesc_f16_f32(BM, p.UW);
            const uint32_t idesc2 = umma_idesc_f16_f32(BM, p.N2);
            const uint32_t hi128 = static_cast<uint32_t>(umma_desc_sw128(0) >> 32);
            auto lo_of = [](uint32_t addr) { return ((addr & 0x3ffffu) >> 4) | 0x10000u; };
            bool failed = false;
            if (T > 0) failed |= !mbar_wait(w_full_bar, 0u, abort_flag);
            for (int step = 0; step < U + DUAL_LAG; ++step) {
                if (step < U) {
                    // GEMM 1 of unit `step`: 128 pixels x UW channels of y
                    const int it = step / p.H, h = step - it * p.H;
                    const int s = step % p.ys, sa = it % p.sa;
                    if (h == 0) failed |= !mbar_wait(a_full_bar(sa), static_cast<uint32_t>(it / p.sa) & 1u, abort_flag);
                    failed |= !mbar_wait(acc1_empty_bar(s), (static_cast<uint32_t>(step / p.ys) & 1u) ^ 1u, abort_flag);
                    tc_fence_after();
                    for (int kb = 0; kb < p.kb1; ++kb)
                        umma_f16_kblock(tmem_base + static_cast<uint32_t>(s * p.UW),
                                        lo_of(a_base + static_cast<uint32_t>(sa) * a_stage_bytes + static_cast<uint32_t>(kb) * A_STAGE_BYTES), hi128,
                                        lo_of(w1_base + static_cast<uint32_t>(kb) * w1_kb_bytes + static_cast<uint32_t>(h * p.UW) * 128u), hi128,
                                        idesc1, static_cast<uint32_t>(kb != 0));
                    umma_commit(acc1_full_bar(s));
                    if (h == p.H - 1) umma_commit(a_empty_bar(sa));       // the x tile is free once these MMAs have read it
                }
                if (step >= DUAL_LAG) {
                    // GEMM 2, the k-blocks (one per panel) that unit `v` of y contributes: A = the finished y slot
                    const int v = step - DUAL_LAG;
                    const int jt = v / p.H, hh = v - jt * p.H;
                    const int s = v % p.ys, b = jt & 1;
                    if (hh == 0) failed |= !mbar_wait(acc2_empty_bar(b), (static_cast<uint32_t>(jt >> 1) & 1u) ^ 1u, abort_flag);
                    failed |= !mbar_wait(y_done_bar(s), static_cast<uint32_t>(v / p.ys) & 1u, abort_flag);
                    tc_fence_after();
                    for (int j = 0; j < p.UP; ++j)
                        umma_f16_kblock(tmem_base + static_cast<uint32_t>(p.acc2_col + b * p.acc2_stride),
                                        lo_of(y_base + static_cast<uint32_t>(s) * y_slot_bytes + static_cast<uint32_t>(j) * SUB_BYTES), hi128,
                                        lo_of(w2_base + static_cast<uint32_t>(hh * p.UP + j) * w2_kb_bytes), hi128, idesc2,
                                        static_cast<uint32_t>((hh | j) != 0));
                    umma_commit(y_free_bar(s));
                    if (hh == p.H - 1) umma_commit(acc2_full_bar(b));
                }
            }
            if (failed) atomicExch(p.status, STATUS_WAIT_DUAL);
        }
        __syncwarp();
    } else if (warp < STORE_WARP) {
        // ------------------------------------------------------------------ epilogue (both layers)
        const int lane_group = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row = lane_group * 32 + lane;
        const uint32_t row_xor = static_cast<uint32_t>(row & 7);
        {
            float* bias_f = reinterpret_cast<float*>(smem_raw + bias_off);
            for (int i = threadIdx.x - 64; i < p.K1 + p.N2; i += EPI_WARPS * 32) {
                const __half* src = i < p.K1 ? p.bias1 : p.bias2;
                bias_f[i] = src != nullptr ? __half2float(src[i < p.K1 ? i : i - p.K1]) : 0.f;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        }
        ConvParams q1, q2;          // what the shared epilogue code reads of its parameter block
        q1.scale = nullptr; q1.act = p.act1;
        q2.scale = nullptr; q2.act = p.act2;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        // activation as a template argument for the common ones, as in the single-layer kernels (same code, same bits)
        const int act1_t = (p.act1 == 0 || p.act1 == 1 || p.act1 == 3 || p.act1 == 5) ? p.act1 : 2;
        const int act2_t = (p.act2 == 0 || p.act2 == 1 || p.act2 == 3 || p.act2 == 5) ? p.act2 : 2;
        bool ok = true;
        auto second = [&](int j) {       // epilogue of the second layer for tile j of this CTA
            const int b = j & 1;
            if (!mbar_wait<EPI_BACKOFF_NS>(z_free_bar, (static_cast<uint32_t>(j) & 1u) ^ 1u, abort_flag) ||
                !mbar_wait<EPI_BACKOFF_NS>(acc2_full_bar(b), static_cast<uint32_t>(j >> 1) & 1u, abort_flag)) {
                if (lane == 0) atomicExch(p.status, STATUS_WAIT_DUAL);
                ok = false;
                return;
            }
            tc_fence_after();
            const uint32_t t = t_lane + static_cast<uint32_t>(p.acc2_col + b * p.acc2_stride);
            const uint32_t srow = z_base + static_cast<uint32_t>(row) * 128u;
            if (act2_t == 0) epilogue_rows<0, false>(q2, t, srow, row_xor, bias2_s, 0, p.N2, group);
            else if (act2_t == 1) epilogue_rows<1, false>(q2, t, srow, row_xor, bias2_s, 0, p.N2, group);
            else if (act2_t == 3) epilogue_rows<3, false>(q2, t, srow, row_xor, bias2_s, 0, p.N2, group);
            else if (act2_t == 5) epilogue_rows<5, false>(q2, t, srow, row_xor, bias2_s, 0, p.N2, group);
            else epilogue_rows<2, false>(q2, t, srow, row_xor, bias2_s, 0, p.N2, group);
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(acc2_empty_bar(b));
                mbar_arrive(z_done_bar);
            }
        };
        int u = 0;
        for (int it = 0; ok && it < T; ++it) {
            for (int h = 0; ok && h < p.H; ++h, ++u) {
                const int s = u % p.ys;
                const uint32_t par = static_cast<uint32_t>(u / p.ys) & 1u;
                const bool got = p.has_res ? mbar_wait<EPI_BACKOFF_NS>(res_full_bar(s), par, abort_flag)
                                           : mbar_wait<EPI_BACKOFF_NS>(y_free_bar(s), par ^ 1u, abort_flag);
                if (!got || !mbar_wait<EPI_BACKOFF_NS>(acc1_full_bar(s), par, abort_flag)) {
                    if (lane == 0) atomicExch(p.status, STATUS_WAIT_DUAL);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t t = t_lane + static_cast<uint32_t>(s * p.UW);
                const uint32_t srow = y_base + static_cast<uint32_t>(s) * y_slot_bytes + static_cast<uint32_t>(row) * 128u;
                const int variant = act1_t * 2 + (p.has_res ? 1 : 0);
                switch (variant) {
                    case 0: epilogue_rows<0, false>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 1: epilogue_rows<0, true>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 2: epilogue_rows<1, false>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 3: epilogue_rows<1, true>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 4: epilogue_rows<2, false>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 5: epilogue_rows<2, true>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 6: epilogue_rows<3, false>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 7: epilogue_rows<3, true>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    case 10: epilogue_rows<5, false>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                    default: epilogue_rows<5, true>(q1, t, srow, row_xor, bias1_s, h * p.UW, p.UW, group); break;
                }
                tc_fence_before();
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(acc1_empty_bar(s));
                    mbar_arrive(y_done_bar(s));
                }
            }
            if (ok && it >= 1) second(it - 1);
        }
        if (ok && T > 0) second(T - 1);
    } else {
        // ------------------------------------------------------------------ store warp
        if (elect_one()) {
            const unsigned long long pol_y = (p.hints & 4) ? l2_policy_evict_last() : 0ull;
            const unsigned long long pol_z = (p.hints & 8) ? l2_policy_evict_last() : 0ull;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            auto store_z = [&](int j) {
                if (!mbar_wait<EPI_BACKOFF_NS>(z_done_bar, static_cast<uint32_t>(j) & 1u, abort_flag)) {
                    atomicExch(p.status, STATUS_WAIT_DUAL);
                    ok = false;
                    return;
                }
                for (int c = 0; c < p.zp; ++c) tma_store_2d(&tmap_z, z_base + static_cast<uint32_t>(c) * SUB_BYTES, c * 64, tile_row0(j), pol_z);
                tma_store_commit();
                tma_store_wait_read();
                mbar_arrive(z_free_bar);
            };
            int u = 0;
            for (int it = 0; ok && it < T; ++it) {
                const int m0 = tile_row0(it);
                for (int h = 0; ok && h < p.H; ++h, ++u) {
                    const int s = u % p.ys;
                    if (!mbar_wait<EPI_BACKOFF_NS>(y_done_bar(s), static_cast<uint32_t>(u / p.ys) & 1u, abort_flag)) {
                        atomicExch(p.status, STATUS_WAIT_DUAL);
                        ok = false;
                        break;
                    }
                    for (int j = 0; j < p.UP; ++j)
                        tma_store_2d(&tmap_y, y_base + static_cast<uint32_t>(s) * y_slot_bytes + static_cast<uint32_t>(j) * SUB_BYTES,
                                     h * p.UW + j * 64, m0, pol_y);
                    tma_store_commit();
                    tma_store_wait_read();
                    mbar_arrive(y_free_bar(s));
                }
                if (ok && it >= 1) store_z(it - 1);
            }
            if (ok && T > 0) store_z(T - 1);
            tma_store_wait_read();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512u);
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
    // Called by fvm_init() once per device, with that device current and under the library's mutex. The driver entry
    // points are looked up once per process; the shared-memory opt-in is a per-device attribute of the kernel and is
    // set for every device that is initialised.
    if (!g_encode_tiled || !g_encode_im2col) {
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
    }
    if (cudaFuncSetAttribute(conv_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess ||
        cudaFuncSetAttribute(conv_streamk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess ||
        cudaFuncSetAttribute(conv_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(conv_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(conv_dual_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
        return FVM_ERR_SETUP;
    return FVM_OK;
}

// How many CTA pairs (clusters of two, one CTA per SM) the device runs at once: the pair kernel's grid never exceeds
// it, so that every pair is resident from the start. 0 if clusters cannot be launched here.
int conv_pair_capacity() {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(CONV_THREADS);
    cfg.dynamicSmemBytes = 227 * 1024;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, conv_pair_kernel, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

int encode_tiled_f16(CUtensorMap* map, const void* ptr, int rank, const unsigned long long* dims,
                     const unsigned long long* strides_bytes, const unsigned* box, bool swizzle128) {
    if (!g_encode_tiled || rank < 1 || rank > 5) return FVM_ERR_SETUP;
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], es[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        es[i] = 1;
        if (i + 1 < rank) st[i] = strides_bytes[i];
    }
    const CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(ptr),
                                      d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FVM_OK : FVM_ERR_TMAP;
}

// Shared-memory plan for an output-channel tile of BN: staging buffers for the residual/output tiles first (3 if the
// main loop still gets enough stages, else 2), then the zero-padded bias copy, the rest goes to the A/B pipeline.
struct SmemPlan {
    int stages, nepi, nacc;
    size_t bytes;
};
static bool plan_smem(int BN, int MT, int kblocks, int K, bool tapk, bool bres, SmemPlan* out, uint32_t halo_bytes = 0,
                      bool pair = false) {
    const int n_tiles = (K + BN - 1) / BN;
    // halo mode (halo_bytes > 0): the activations live in two staged input patches, the stages carry weights only
    const uint32_t stage_bytes = (halo_bytes ? 0u : static_cast<uint32_t>(MT) * A_STAGE_BYTES) +
                                 ((tapk || bres) ? 0u : static_cast<uint32_t>(pair ? BN / 2 : BN) * BK * 2);   // a pair CTA holds half of B
    const uint32_t bres_bytes = tapk ? static_cast<uint32_t>(kblocks) * BN * BK * 2   // 8 x 16 B or 4 x 32 B per row
                                     : (bres ? static_cast<uint32_t>(kblocks) * BN * BK * 2 : 0u);
    const uint32_t epi_bytes = static_cast<uint32_t>(MT * ((BN + 63) / 64)) * SUB_BYTES;
    const uint32_t bias_bytes = (static_cast<uint32_t>(n_tiles * BN) * 4 + 15u) & ~15u;   // fp32 copy of the bias
    if (bias_bytes > MAX_BIAS_BYTES) return false;
    const uint32_t fixed = 1024 + 8 * NUM_BARRIERS + MISC_BYTES + bias_bytes + bres_bytes + 2 * halo_bytes;
    const uint32_t total = 227 * 1024;
    // deep reductions reach the epilogue rarely: they may run on a single staging buffer and give the rest to the pipeline
    const int floor_epi = kblocks >= 16 ? 1 : 2;
    if (fixed + static_cast<uint32_t>(floor_epi) * epi_bytes + 2 * stage_bytes > total) return false;
    const uint32_t budget = total - fixed;
    // All epilogue warps work on one tile at a time, so two accumulators already overlap a tile's epilogue with the
    // next tile's MMAs (TMEM is not scarce: up to 4 are used when they fit the 512 columns) and three staging buffers
    // cover "residual arriving / being combined / being stored"; the rest of the shared memory goes to the pipeline.
    int acc_stride = 32;
    while (acc_stride < MT * BN) acc_stride <<= 1;
    if (acc_stride > 256) return false;    // at least two accumulator buffers in the 512 TMEM columns
    const int nacc = 512 / acc_stride < MAX_ACC ? 512 / acc_stride : MAX_ACC;
    const int min_stages = 4;   // loads in flight span tiles of this persistent CTA, also when one tile has a single k-block
    int nepi = kblocks <= 2 ? 4 : 3;
    while (nepi > floor_epi &&
           static_cast<uint32_t>(nepi) * epi_bytes + static_cast<uint32_t>(min_stages) * stage_bytes > budget)
        --nepi;
    int stages = stage_bytes ? static_cast<int>((budget - static_cast<uint32_t>(nepi) * epi_bytes) / stage_bytes) : 2;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    out->nacc = nacc;
    out->stages = stages;
    out->nepi = nepi;
    out->bytes = fixed + static_cast<size_t>(stages) * stage_bytes + static_cast<size_t>(nepi) * epi_bytes;
    return true;
}

// Picks the output-channel tile. A single tile over all of K (any multiple of 16 up to 256) reads A once; when K is
// split, tiles must be multiples of 64 channels because the output leaves in 64-channel TMA boxes. Among the
// candidates that fit shared memory the best (wave efficiency x useful-column fraction) wins, larger tiles first;
// a deep reduction (many k-blocks) additionally wants at least 3 pipeline stages.
static int pick_bn(int m_tiles, int K, int kblocks, bool tapk, int sms) {
    const int Kp = (K + 31) / 32 * 32;
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
        if (!plan_smem(bn, 1, kblocks, K, tapk, false, &sp)) continue;
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

static int launch_conv_kernel(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const CUtensorMap& tmap_r,
                              const CUtensorMap& tmap_y, const ConvParams& p, int grid, size_t smem, cudaStream_t stream);

// Stride-2 stem over an 8-channel input held as two column-parity planes per image row (x: [N][H][2][W/2][8], the
// layout fvm_input_nhwc8_split_f32 writes): y = act(conv(x, w) + bias), w [K][R][S][8], symmetric padding, no residual.
int stem_s2_launch(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int K, int R, int S,
                   int ph, int pw, long long ldy, int act, cudaStream_t stream) {
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    if (!x || !w || !y) return FVM_ERR_ARG;
    if (N <= 0 || H <= 0 || W <= 0 || (W & 1) || K <= 0 || (K & 7) || K > 256 || R <= 0 || S <= 0 || R > 8 || S > 8)
        return FVM_ERR_ARG;
    if (ph < 0 || pw < 0 || ph >= R || pw >= S || (ldy & 7) || ldy < K || act < 0 || act > 6) return FVM_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(bias) & 15))
        return FVM_ERR_ARG;
    const int P = (H + 2 * ph - R) / 2 + 1, Q = (W + 2 * pw - S) / 2 + 1;
    if (H + 2 * ph < R || W + 2 * pw < S || P <= 0 || Q <= 0) return FVM_ERR_ARG;
    const long long M_ll = static_cast<long long>(N) * P * Q;
    if (M_ll > 0x7fffff00ll) return FVM_ERR_ARG;

    ConvParams p;
    memset(&p, 0, sizeof(p));
    p.M = static_cast<int>(M_ll);
    p.K = K; p.C = 8; p.R = R; p.S = S; p.P = P; p.Q = Q;
    p.sh = p.sw = 2; p.ph = ph; p.pw = pw; p.dh = p.dw = 1;
    p.cchunks = 1;
    p.taps = R * S;
    const int RP = (R + 1) & ~1;                   // rows of taps, rounded up to pairs (the extra row has zero weights)
    p.stem_taps = RP * S;
    p.kblocks = p.stem_taps / 2;                  // MMAs per tile (reporting only)
    p.BN = (K + 31) / 32 * 32;
    p.n_tiles = 1;
    p.div_ntiles = fastdiv_init(1);
    p.nsub = (p.BN + 63) / 64;
    p.mt = 1;
    p.halo = 2;
    p.bres = 1;
    p.tiles_x = (Q + HALO_TW - 1) / HALO_TW;
    p.tiles_y = (P + HALO_TH - 1) / HALO_TH;
    p.div_txy = fastdiv_init(static_cast<uint32_t>(p.tiles_x * p.tiles_y));
    p.div_tx = fastdiv_init(static_cast<uint32_t>(p.tiles_x));
    p.div_pq = fastdiv_init(static_cast<uint32_t>(P) * Q);
    p.div_q = fastdiv_init(static_cast<uint32_t>(Q));
    p.m_tiles = N * p.tiles_x * p.tiles_y;
    // plane columns a tap column s reaches: (s - pw - parity) / 2 relative to the output column
    auto xoff = [&](int s_) { const int d = s_ - pw, par = d & 1; return (d - par) / 2; };
    p.stem_xlo = xoff(0);
    const int PW = (HALO_TW + xoff(S - 1) - p.stem_xlo + 7) & ~7;      // staged plane columns (rows of whole 128 bytes)
    const int PR = 2 * (HALO_TH - 1) + RP;                  // staged input rows (incl. the zero-weight tap row)
    p.stem_prow = static_cast<uint32_t>(2 * PW * 16);
    p.htx = static_cast<uint32_t>(PR) * p.stem_prow;
    p.hbytes = (p.htx + 127u) & ~127u;
    p.nh = 3;
    p.act = act;
    p.has_res = 0;
    p.bias = static_cast<const __half*>(bias);
    p.scale = nullptr;
    p.status = st->status_dev;
    p.bias_elems = p.BN;
    p.acc_stride = 32;
    while (p.acc_stride < p.BN) p.acc_stride <<= 1;
    p.nacc = 512 / p.acc_stride >= 4 ? 4 : 2;
    p.tmem_cols = p.nacc * p.acc_stride;
    p.stages = 2;                                  // unused: the stages are empty in this mode
    const uint32_t bres_bytes = static_cast<uint32_t>(p.stem_taps) * p.BN * 16u;
    const uint32_t epi_bytes = static_cast<uint32_t>(p.nsub) * SUB_BYTES;
    uint32_t fixed = 1024 + 8 * NUM_BARRIERS + MISC_BYTES + ((static_cast<uint32_t>(p.BN) * 4 + 15u) & ~15u) +
                     bres_bytes + static_cast<uint32_t>(p.nh) * p.hbytes;
    if (fixed + 2 * epi_bytes > 227u * 1024) {       // wide tiles: two staged patches instead of three
        p.nh = 2;
        fixed -= p.hbytes;
    }
    p.nepi = 4;
    while (p.nepi > 2 && fixed + static_cast<uint32_t>(p.nepi) * epi_bytes > 227u * 1024) --p.nepi;
    if (fixed + static_cast<uint32_t>(p.nepi) * epi_bytes > 227u * 1024) return FVM_ERR_ARG;
    size_t smem = fixed + static_cast<size_t>(p.nepi) * epi_bytes;
    if (smem < 120 * 1024) smem = 120 * 1024;

    CUtensorMap tmap_a, tmap_b, tmap_y;
    {
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(Q), static_cast<cuuint64_t>(P),
                              static_cast<cuuint64_t>(N)};
        cuuint32_t box[4] = {64, HALO_TW, HALO_TH, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        cuuint64_t ystr[3] = {static_cast<cuuint64_t>(ldy) * 2, static_cast<cuuint64_t>(Q) * ldy * 2,
                              static_cast<cuuint64_t>(P) * Q * ldy * 2};
        if (g_encode_tiled(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, y, dims, ystr, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return FVM_ERR_TMAP;
    }
    {
        // weights [K][R*S][8]: one tap of all output channels per load, 16-byte rows, no swizzle
        cuuint64_t dims[3] = {8, static_cast<cuuint64_t>(R * S), static_cast<cuuint64_t>(K)};
        cuuint64_t strides[2] = {16, static_cast<cuuint64_t>(R) * S * 16};
        cuuint32_t box[3] = {8, 1, static_cast<cuuint32_t>(p.BN)};
        cuuint32_t estr[3] = {1, 1, 1};
        if (g_encode_tiled(&tmap_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return FVM_ERR_TMAP;
    }
    {
        // input as (channel 8, plane column W/2, plane 2, row H, image N); a box = the input of one output patch
        cuuint64_t dims[5] = {8, static_cast<cuuint64_t>(W / 2), 2, static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(N)};
        cuuint64_t strides[4] = {16, static_cast<cuuint64_t>(W / 2) * 16, static_cast<cuuint64_t>(W) * 16,
                                 static_cast<cuuint64_t>(H) * W * 16};
        cuuint32_t box[5] = {8, static_cast<cuuint32_t>(PW), 2, static_cast<cuuint32_t>(PR), 1};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        if (g_encode_tiled(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(x), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return FVM_ERR_TMAP;
    }
    int grid = p.m_tiles < st->sms ? p.m_tiles : st->sms;
    return launch_conv_kernel(tmap_a, tmap_b, tmap_y, tmap_y, p, grid, smem, stream);
}

int conv2d_launch(const void* x, const void* w, const void* bias, const void* res, const float* scale, void* y, int N,
                  int H, int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                  long long ldx, long long ldy, long long ldr, int act, int force_bn, int ph_hi, int pw_hi,
                  cudaStream_t stream, int w_per_image, int gsg, int gsk) {
    // ph / pw pad the top / left; ph_hi / pw_hi the bottom / right (negative: same as top / left)
    if (ph_hi < 0) ph_hi = ph;
    if (pw_hi < 0) pw_hi = pw;
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    if (!x || !w || !y) return FVM_ERR_ARG;
    // force_bn: low 16 bits = output-channel tile (0 = choose), bits 16..23 = sub-tiles per tile (0 = choose),
    // bits 24..25 = weight-resident mode (0 = choose, 1 = on, 2 = off), bits 26..27 = halo mode, bits 28..29 = stream-K
    // (same coding), bit 30 = CTA pairs (conv_pair_kernel) on
    int force_pair = force_bn > 0 ? ((force_bn >> 30) & 1) : 0;
    const bool free_choice = force_bn <= 0;
    const int force_sk = force_bn > 0 ? ((force_bn >> 28) & 3) : 0;
    const int force_halo = force_bn > 0 ? ((force_bn >> 26) & 3) : 0;
    const int force_bres = force_bn > 0 ? ((force_bn >> 24) & 3) : 0;
    const int force_mt = force_bn > 0 ? ((force_bn >> 16) & 0xff) : 0;
    force_bn = force_bn > 0 ? (force_bn & 0xffff) : 0;
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || R <= 0 || S <= 0) return FVM_ERR_ARG;
    if ((C & 7) || (K & 7) || (ldx & 7) || (ldy & 7) || (res && (ldr & 7))) return FVM_ERR_ARG;
    if (sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || ph < 0 || pw < 0) return FVM_ERR_ARG;
    if (ldx < C || ldy < K || (res && ldr < K)) return FVM_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(res) & 15) ||
        (reinterpret_cast<uintptr_t>(bias) & 15) || (reinterpret_cast<uintptr_t>(scale) & 15))
        return FVM_ERR_ARG;      // bias is read as 16-byte vectors, scale as float4
    if (act < 0 || act > 6) return FVM_ERR_ARG;
    const int P = (H + ph + ph_hi - dh * (R - 1) - 1) / sh + 1;
    const int Q = (W + pw + pw_hi - dw * (S - 1) - 1) / sw + 1;
    if (P <= 0 || Q <= 0) return FVM_ERR_ARG;
    const long long M_ll = static_cast<long long>(N) * P * Q;
    if (M_ll > 0x7fffff00ll) return FVM_ERR_ARG;

    ConvParams p;
    memset(&p, 0, sizeof(p));
    p.M = static_cast<int>(M_ll);
    p.K = K; p.C = C; p.R = R; p.S = S; p.P = P; p.Q = Q;
    p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
    p.cchunks = (C + BK - 1) / BK;
    if (gsg > 0) {
        // Grouped convolution as block-diagonal dense convolutions over "super-groups": the channels are cut into runs
        // of gsg input / gsk output channels (whole groups; gsk a multiple of 64 so that output tiles and their
        // 64-channel store boxes never straddle a run, the last run may be short), and w is [K][R*S][gsg] with zeros
        // outside each output channel's own group. An n-tile then reads only the input channels of its run.
        if (w_per_image || (gsg & 7) || gsk <= 0 || (gsk < K && (gsk & 63)) || gsg > C || force_sk == 1 || force_pair ||
            force_mt > 1)
            return FVM_ERR_ARG;
        if ((static_cast<long long>(C) + gsg - 1) / gsg != (static_cast<long long>(K) + gsk - 1) / gsk) return FVM_ERR_ARG;
        p.gsg = gsg;
        p.gsk = gsk;
        p.div_gsk = fastdiv_init(static_cast<uint32_t>(gsk));
        p.cchunks = (gsg + BK - 1) / BK;
        if (force_bn <= 0) force_bn = gsk >= K ? 0 : (gsk % 256 == 0 ? 256 : (gsk % 128 == 0 ? 128 : 64));
        if (force_bn > 0 && gsk < K && gsk % force_bn) return FVM_ERR_ARG;
    }
    p.kblocks = R * S * p.cchunks;
    p.m_tiles = (p.M + BM - 1) / BM;
    p.taps = R * S;
    if (w_per_image) {
        // w is [N][K][C]: 1x1 stride-1 only, tiles never straddle images
        if (R != 1 || S != 1 || sh != 1 || sw != 1 || ph || pw || ph_hi || pw_hi || force_mt > 2 || force_halo == 1 ||
            force_bres == 1 || force_sk == 1)
            return FVM_ERR_ARG;
        p.wb = 1;
        p.wb_tpi = (P * Q + BM - 1) / BM;
        p.div_tpi = fastdiv_init(static_cast<uint32_t>(p.wb_tpi));
        p.m_tiles = N * p.wb_tpi;
    }
    // Tap-packed mode for 8-channel inputs (zero-padded RGB stems): 8 taps per k-block instead of one tap with 56 of
    // its 64 channels empty. Needs all output channels in one tile (the weights stay resident in shared memory).
    {
        const int Kp16 = (K + 31) / 32 * 32;   // tiles are multiples of 32 channels
        SmemPlan tp;
        const int tpk = (C == 8 || C == 16) ? BK / C : 1;      // taps per k-block in tap-packed mode
        p.tapk = (!gsg && (C == 8 || C == 16) && R * S > 1 && Kp16 <= 256 && (force_bn <= 0 || force_bn >= Kp16) &&
                  plan_smem(Kp16, 1, (R * S + tpk - 1) / tpk, K, true, false, &tp)) ? C : 0;
        if (p.tapk) {
            p.kblocks = (R * S + tpk - 1) / tpk;
            force_bn = Kp16;
        }
    }
    // Halo mode for 3x3 stride-1 convolutions (dilation up to 4): an m-tile is a 16 x 8 patch of output pixels of one
    // image. Chosen when few patch pixels fall outside the image (they are computed and clipped by the store).
    uint32_t halo_bytes = 0;
    if (!p.tapk && R == 3 && S == 3 && sh == 1 && sw == 1 && dh == dw && dh <= 4 && force_halo != 2 && force_mt <= 1 && !force_pair) {
        const int ty = (P + HALO_TH - 1) / HALO_TH, tx = (Q + HALO_TW - 1) / HALO_TW;
        const double eff = static_cast<double>(P) * Q / (static_cast<double>(ty) * tx * BM);
        // by default only for inputs of one 64-channel chunk: there the taps are accumulated in the same order as in
        // im2col mode (bit-identical results), and the measured gain is largest (at 56 x 56, where an eighth of the
        // patch rows fall outside the image: 23.7 us against 32.6 us for 64 -> 64 at batch 64)
        if (force_halo == 1 || (eff >= 0.85 && p.cchunks == 1)) {
            p.halo = 1;
            p.halo_rows = HALO_TH + (R - 1) * dh;
            p.nh = 2;
            p.tiles_x = tx;
            p.tiles_y = ty;
            p.div_txy = fastdiv_init(static_cast<uint32_t>(tx * ty));
            p.div_tx = fastdiv_init(static_cast<uint32_t>(tx));
            p.m_tiles = N * ty * tx;
            halo_bytes = static_cast<uint32_t>(p.halo_rows * HALO_PITCH) * 128u;
            p.hbytes = p.htx = halo_bytes;
        }
    }
    if (force_halo == 1 && !p.halo) return FVM_ERR_ARG;
    // CTA pairs by default where the weight tiles are what the SMs pull most (at most four 128-pixel tiles per SM: the
    // 28x28 and smaller maps of a ResNet at batch 64; measured there: 10-25 % faster than the best single-CTA tile).
    // Tile width from the same measurements: all of K (up to 256) for deep reductions without a residual, else 128.
    static const int auto_pairs = [] { const char* v = getenv("FVM_B200_PAIR"); return (v && v[0] == '0') ? 0 : 1; }();
    if (free_choice && auto_pairs && !gsg && !p.tapk && !p.halo && !p.wb && st->pair_clusters > 0 && C >= 24 && K >= 64 &&
        p.m_tiles <= 4 * st->sms) {
        const int bn = (K <= 128 || (K <= 256 && !res && p.kblocks >= 8)) ? (K + 31) / 32 * 32 : 128;
        SmemPlan tp;
        if (plan_smem(bn, 1, p.kblocks, K, false, false, &tp, 0, true)) {
            force_pair = 1;
            force_bn = bn;
        }
    }
    p.BN = force_bn > 0 ? force_bn : pick_bn(p.m_tiles, K, p.kblocks, false, st->sms);
    if (p.BN < 32 || p.BN > 256 || (p.BN & 31)) return FVM_ERR_ARG;
    p.n_tiles = (K + p.BN - 1) / p.BN;
    p.div_ntiles = fastdiv_init(static_cast<uint32_t>(p.n_tiles));
    if (p.n_tiles > 1 && (p.BN & 63)) return FVM_ERR_ARG;   // split K only in whole 64-channel store boxes
    p.im2col = !(R == 1 && S == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0 && ph_hi == 0 && pw_hi == 0);
    p.act = act;
    // Tile order: a 1x1 stride-1 layer without residual whose input is larger than half of the L2 and at least four
    // times wider than its output (the first convolution of a bottleneck block, reading the previous block's output)
    // walks its m-tiles from the last to the first: the kernel before it wrote that tensor front to back, so the tail
    // is what the L2 still holds (measured inside a ResNet-50 forward at batch 64: 27.6 -> 21.8 us for 256 -> 64 at 56x56).
    {
        static const int rev_rule = [] { const char* v = getenv("FVM_B200_REVERSE"); return (v && v[0] == '0') ? 0 : 1; }();
        if (rev_rule && R == 1 && S == 1 && sh == 1 && sw == 1 && !res && C >= 4 * K &&
            static_cast<long long>(p.M) * ldx * 2 > 64ll * 1024 * 1024)
            p.rev = 1;
    }
    p.has_res = res != nullptr;
    p.bias = static_cast<const __half*>(bias);
    p.scale = scale;
    p.status = st->status_dev;
    p.div_pq = fastdiv_init(static_cast<uint32_t>(P) * Q);
    p.div_q = fastdiv_init(static_cast<uint32_t>(Q));
    p.nsub = (p.BN + 63) / 64;
    // Measured on B200: larger tiles did not pay for themselves on the layers tried (fewer, larger hand-offs but less
    // overlap between the roles), so the default stays at one sub-tile; the host's per-layer tuning may force more.
    p.mt = force_mt > 0 ? force_mt : 1;
    if (p.wb && force_mt == 0 && p.kblocks <= 3 && p.BN <= 64 && p.m_tiles >= 8 * st->sms) {
        // short reductions into narrow tiles on large maps (measured: 1x1 48->24 at 190x190, N = 64: 143 us with
        // 128-pixel tiles, 81 us with 256-pixel tiles): halve the per-tile hand-offs when the plan still fits
        SmemPlan tp;
        if (plan_smem(p.BN, 2, p.kblocks, K, false, false, &tp)) p.mt = 2;
    }
    if (p.mt != 1 && p.mt != 2 && p.mt != 4) return FVM_ERR_ARG;
    if (p.wb) {
        p.wb_tpi = (P * Q + BM * p.mt - 1) / (BM * p.mt);
        p.div_tpi = fastdiv_init(static_cast<uint32_t>(p.wb_tpi));
        p.m_tiles = N * p.wb_tpi;
    }
    if (!p.halo && !p.wb) p.m_tiles = (p.M + BM * p.mt - 1) / (BM * p.mt);
    p.a_rows = BM * p.mt < 256 ? BM * p.mt : 256;
    p.a_loads = BM * p.mt / p.a_rows;
    // CTA pairs (conv_pair_kernel): on request only, plain mode only
    if (force_pair) {
        if (p.tapk || p.halo || p.wb || p.mt != 1 || force_bres == 1 || force_sk == 1 || st->pair_clusters <= 0)
            return FVM_ERR_ARG;
        p.pair = 1;
        p.m_tiles = (p.M + 2 * BM - 1) / (2 * BM);
    }

    // Weight-resident mode: the weight tile of a CTA's n-tile (all k-blocks) is loaded once and kept; the stages then
    // carry activations only, so more tiles' worth of loads are in flight and the weights are not re-read from L2 for
    // every tile. Used when the tile fits in 96 KB, every CTA gets at least two tiles, and the grid can be made a
    // multiple of the n-tile count.
    // Stream-K (see conv_streamk_kernel): on request only.
    {
        const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
        const long long units = tiles * p.kblocks;
        const bool can = !p.tapk && !p.halo && !p.wb && !p.pair && !gsg && p.mt == 1 && force_bres != 1 && st->sk_part != nullptr && p.kblocks >= 2 &&
                         units >= st->sms && units < 0x7fffffffll &&
                         static_cast<size_t>(st->sms) * BM * p.BN <= st->sk_floats;
        if (force_sk == 1 && !can) return FVM_ERR_ARG;
        p.sk = (can && force_sk == 1) ? 1 : 0;     // only on request: the host's per-layer timing decides
        if (p.sk) {
            p.sk_units = static_cast<uint32_t>(units);
            p.div_kb = fastdiv_init(static_cast<uint32_t>(p.kblocks));
            p.sk_part = st->sk_part;
            p.sk_flags = st->sk_flags;
        }
    }
    SmemPlan sp;
    p.bres = 0;
    if (!p.sk && !p.wb && !p.tapk && !p.pair && force_bres != 2 && p.n_tiles <= st->sms) {
        const long long wbytes = static_cast<long long>(p.kblocks) * p.BN * BK * 2;
        const int cta_per_n = st->sms / p.n_tiles;
        const bool worth = p.m_tiles >= 2 * cta_per_n;
        SmemPlan rp;
        if (wbytes <= 96 * 1024 && (worth || force_bres == 1) &&
            plan_smem(p.BN, p.mt, p.kblocks, K, false, true, &rp, halo_bytes) &&
            (rp.stages >= 4 || p.halo || force_bres == 1))
            p.bres = 1;
    }
    if (force_bres == 1 && !p.bres) return FVM_ERR_ARG;
    if (!plan_smem(p.BN, p.mt, p.kblocks, K, p.tapk != 0, p.bres != 0, &sp, halo_bytes, p.pair != 0)) return FVM_ERR_ARG;
    p.bias_elems = p.n_tiles * p.BN;
    p.stages = sp.stages;
    p.nepi = sp.nepi;
    p.nacc = sp.nacc;
    p.acc_stride = 32;
    while (p.acc_stride < p.mt * p.BN) p.acc_stride <<= 1;
    p.tmem_cols = p.nacc * p.acc_stride;   // a power of two between 64 and 512
    // Always request more than half of an SM's shared memory: at most one CTA per SM, so the TMEM request of a CTA
    // never waits on a co-resident CTA of the same kernel.
    size_t smem = sp.bytes;
    if (smem < 120 * 1024) smem = 120 * 1024;

    // L2 eviction hints (performance only). A convolution with a fused residual closes a block: its residual operand is
    // dead after it (evict first) and its output is read twice soon, by the next block's first layer and as that block's
    // residual (evict last, if it can stay: at most 112 MB against the 126 MB L2). The input is fetched evict-first only
    // where the kernel reads each element once or in one burst (staged patches; a 1x1 layer with a single n-tile that
    // closes a block): im2col loads and several n-tiles come back to the same lines and must find them in the L2
    // (measured: hints on im2col inputs cost DeepLabV3 5 %). Inside a ResNet-50 forward at batch 64 stage 1 (103 MB
    // tensors) ends 5-10 us earlier, 1.100 -> 1.08 ms per forward; ConvNeXt-T 1.93 -> 1.89 ms. FVM_B200_L2_HINTS=0: off.
    {
        static const int l2_hints = [] { const char* v = getenv("FVM_B200_L2_HINTS"); return (v && v[0] == '0') ? 0 : 1; }();
        if (l2_hints) {
            if (res) {
                p.hints |= 2;
                if (static_cast<long long>(p.M) * ldy * 2 <= 112ll * 1024 * 1024) p.hints |= 4;
                if (R == 1 && S == 1 && p.n_tiles == 1) p.hints |= 1;
            }
            if (p.halo == 1) p.hints |= 1;
        }
    }
    CUtensorMap tmap_a, tmap_b, tmap_r, tmap_y;
    if (p.halo) {
        // output / residual as (K, Q, P, N): 64-channel x 8-column x 16-row boxes (clipped at the image border)
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(Q), static_cast<cuuint64_t>(P),
                              static_cast<cuuint64_t>(N)};
        cuuint32_t box[4] = {64, HALO_TW, HALO_TH, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        cuuint64_t ystr[3] = {static_cast<cuuint64_t>(ldy) * 2, static_cast<cuuint64_t>(Q) * ldy * 2,
                              static_cast<cuuint64_t>(P) * Q * ldy * 2};
        CUresult r = g_encode_tiled(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, y, dims, ystr, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
        if (res) {
            cuuint64_t rstr[3] = {static_cast<cuuint64_t>(ldr) * 2, static_cast<cuuint64_t>(Q) * ldr * 2,
                                  static_cast<cuuint64_t>(P) * Q * ldr * 2};
            r = g_encode_tiled(&tmap_r, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(res), dims, rstr, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
        } else {
            tmap_r = tmap_y;
        }
    } else if (p.wb) {
        // output / residual as (K, pixel of the image, image): 64-channel x 128-pixel boxes, clipped per image
        const unsigned long long dims[3] = {static_cast<unsigned long long>(K), static_cast<unsigned long long>(P) * Q,
                                            static_cast<unsigned long long>(N)};
        const unsigned box[3] = {64, BM, 1};
        const unsigned long long ystr[2] = {static_cast<unsigned long long>(ldy) * 2, static_cast<unsigned long long>(P) * Q * ldy * 2};
        if (encode_tiled_f16(&tmap_y, y, 3, dims, ystr, box, true) != FVM_OK) return FVM_ERR_TMAP;
        if (res) {
            const unsigned long long rstr[2] = {static_cast<unsigned long long>(ldr) * 2, static_cast<unsigned long long>(P) * Q * ldr * 2};
            if (encode_tiled_f16(&tmap_r, res, 3, dims, rstr, box, true) != FVM_OK) return FVM_ERR_TMAP;
        } else {
            tmap_r = tmap_y;
        }
    } else {
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
        // weights [K][R*S][C] (per-image weights: [N * K][1][C], image n's rows start at n * K)
        const int Cw = gsg > 0 ? gsg : C;      // input channels per weight row
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(Cw), static_cast<cuuint64_t>(R * S),
                              static_cast<cuuint64_t>(K) * (p.wb ? N : 1)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(Cw) * 2, static_cast<cuuint64_t>(R) * S * Cw * 2};
        cuuint32_t box[3] = {static_cast<cuuint32_t>(p.tapk ? p.tapk : BK), 1, static_cast<cuuint32_t>(p.pair ? p.BN / 2 : p.BN)};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = g_encode_tiled(&tmap_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w), dims, strides,
                                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    p.tapk == 8 ? CU_TENSOR_MAP_SWIZZLE_NONE
                                                : (p.tapk == 16 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B),
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
    }
    if (p.halo) {
        // NHWC activation as (C, W, H, N): one box = 64 channels x 16 pixels x (16 + 2*dilation) rows, zero outside
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(N)};
        cuuint64_t strides[3] = {static_cast<cuuint64_t>(ldx) * 2, static_cast<cuuint64_t>(W) * ldx * 2,
                                 static_cast<cuuint64_t>(H) * W * ldx * 2};
        cuuint32_t box[4] = {BK, HALO_PITCH, static_cast<cuuint32_t>(p.halo_rows), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = g_encode_tiled(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(x), dims, strides,
                                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
    } else if (p.wb) {
        const unsigned long long dims[3] = {static_cast<unsigned long long>(C), static_cast<unsigned long long>(P) * Q,
                                            static_cast<unsigned long long>(N)};
        const unsigned long long strides[2] = {static_cast<unsigned long long>(ldx) * 2, static_cast<unsigned long long>(P) * Q * ldx * 2};
        const unsigned box[3] = {BK, static_cast<unsigned>(p.a_rows), 1};
        if (encode_tiled_f16(&tmap_a, x, 3, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
    } else if (!p.im2col) {
        cuuint64_t dims[2] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(p.M)};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldx) * 2};
        cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(p.a_rows)};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = g_encode_tiled(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides,
                                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
    } else {
        // NHWC activation as (C, W, H, N); the filter-window origin moves inside the box
        // [-pad, size + pad - dilation*(taps-1) - 1], stepping by the conv stride; each load adds the tap offset.
        const int up_w = pw_hi - (S - 1) * dw, up_h = ph_hi - (R - 1) * dh;
        if (pw > 128 || ph > 128 || pw_hi > 127 || ph_hi > 127 || up_w < -128 || up_h < -128 || (S - 1) * dw > 255 || (R - 1) * dh > 255)
            return FVM_ERR_ARG;
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(N)};
        cuuint64_t strides[3] = {static_cast<cuuint64_t>(ldx) * 2, static_cast<cuuint64_t>(W) * ldx * 2,
                                 static_cast<cuuint64_t>(H) * W * ldx * 2};
        int lower[2] = {-pw, -ph};
        int upper[2] = {up_w, up_h};
        cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(sw), static_cast<cuuint32_t>(sh), 1};
        CUresult r = g_encode_im2col(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(x), dims, strides,
                                     lower, upper, p.tapk ? p.tapk : BK, static_cast<cuuint32_t>(BM * p.mt), estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     p.tapk == 8 ? CU_TENSOR_MAP_SWIZZLE_NONE
                                                 : (p.tapk == 16 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B),
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
        // Driver releases up to CUDA 13.1 mis-handle im2col maps over tensors smaller than 128 KiB unless bit 21 of
        // the descriptor's second word is cleared (the same correction CUTLASS applies when it builds these maps).
        const unsigned long long bytes = static_cast<unsigned long long>(N) * H * W * ldx * 2;
        if (g_driver_version <= 13010 && bytes < 131072ull)
            reinterpret_cast<uint64_t*>(&tmap_a)[1] &= ~(1ull << 21);
    }

    const long long total_tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
    int grid = static_cast<int>(total_tiles < st->sms ? total_tiles : st->sms);
    if (p.bres) {
        int cta_per_n = st->sms / p.n_tiles;
        if (cta_per_n > p.m_tiles) cta_per_n = p.m_tiles;
        grid = cta_per_n * p.n_tiles;
    }
    if (p.sk) grid = st->sms;       // units >= SMs: every CTA gets at least one k-block
    if (p.pair) grid = 2 * static_cast<int>(total_tiles < st->pair_clusters ? total_tiles : st->pair_clusters);
    return launch_conv_kernel(tmap_a, tmap_b, tmap_r, tmap_y, p, grid, smem, stream);
}

static int launch_conv_kernel(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const CUtensorMap& tmap_r,
                              const CUtensorMap& tmap_y, const ConvParams& p, int grid, size_t smem, cudaStream_t stream) {
    // Programmatic dependent launch: the grid may start (set-up only) while the previous kernel of the stream drains;
    // the kernel itself waits (griddepcontrol.wait) before it touches activations or outputs.
    static int use_pdl = [] { const char* v = getenv("FVM_B200_PDL"); return (v && v[0] == '0') ? 0 : 1; }();
    if (use_pdl || p.pair) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(static_cast<unsigned>(grid));
        cfg.blockDim = dim3(CONV_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attrs[2];
        int na = 0;
        if (use_pdl) {
            attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attrs[na].val.programmaticStreamSerializationAllowed = 1;
            ++na;
        }
        if (p.pair) {       // clusters of two CTAs: blocks 2i and 2i + 1 share a tile
            attrs[na].id = cudaLaunchAttributeClusterDimension;
            attrs[na].val.clusterDim.x = 2;
            attrs[na].val.clusterDim.y = 1;
            attrs[na].val.clusterDim.z = 1;
            ++na;
        }
        cfg.attrs = attrs;
        cfg.numAttrs = static_cast<unsigned>(na);
        const cudaError_t err = p.pair ? cudaLaunchKernelEx(&cfg, conv_pair_kernel, tmap_a, tmap_b, tmap_r, tmap_y, p)
                                : p.sk ? cudaLaunchKernelEx(&cfg, conv_streamk_kernel, tmap_a, tmap_b, tmap_r, tmap_y, p)
                                       : cudaLaunchKernelEx(&cfg, conv_tcgen05_kernel, tmap_a, tmap_b, tmap_r, tmap_y, p);
        if (err == cudaSuccess) {
            count_launch();
            return FVM_OK;
        }
        (void)cudaGetLastError();
        if (p.pair) return FVM_ERR_LAUNCH;
        use_pdl = 0;      // not accepted here (e.g. by an older driver during capture): plain launches from now on
    }
    if (p.sk) conv_streamk_kernel<<<grid, CONV_THREADS, smem, stream>>>(tmap_a, tmap_b, tmap_r, tmap_y, p);
    else conv_tcgen05_kernel<<<grid, CONV_THREADS, smem, stream>>>(tmap_a, tmap_b, tmap_r, tmap_y, p);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------------ chain launch
static bool ranges_overlap(const void* a, size_t na, const void* b, size_t nb) {
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + nb && b0 < a0 + na;
}

// A run of convolutions as one launch of conv_chain_kernel. Layer i may read (as input or residual) the output of an
// earlier layer of the chain, which is recognised by its pointer, shape and row stride; anything else it reads must be
// complete before the launch (stream order). Refused (FVM_ERR_ARG, nothing launched): layers the pair kernel does not
// take (fewer than 24 input channels, per-image weights), more than CHAIN_MAX_EXT_RES residuals that no layer of the
// chain produces, buffers that alias one another in a way the dependency tracking cannot express, more than
// CHAIN_MAX_LAYERS layers.
int conv_chain_launch(const fvm_chain_layer* layers, int n, cudaStream_t stream) {
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    if (!layers || n <= 0 || n > CHAIN_MAX_LAYERS) return FVM_ERR_ARG;
    if (st->pair_clusters <= 0 || !st->chain_flags) return FVM_ERR_ARG;
    static ChainParams cp;      // 28 KB: kept off the stack; guarded by the mutex below
    static std::mutex cp_mutex;
    std::lock_guard<std::mutex> lock(cp_mutex);
    memset(&cp, 0, sizeof(cp));
    cp.n_layers = n;
    int max_bn = 0, max_bias = 0, tiles = 0, flags = 0, n_ext = 0;
    size_t xbytes[CHAIN_MAX_LAYERS], ybytes[CHAIN_MAX_LAYERS];
    for (int i = 0; i < n; ++i) {
        const fvm_chain_layer& a = layers[i];
        ChainLayer& L = cp.L[i];
        if (!a.x || !a.w || !a.y) return FVM_ERR_ARG;
        if (a.N <= 0 || a.H <= 0 || a.W <= 0 || a.C < 24 || a.K <= 0 || a.R <= 0 || a.S <= 0) return FVM_ERR_ARG;
        if ((a.C & 7) || (a.K & 7) || (a.ldx & 7) || (a.ldy & 7) || (a.res && (a.ldr & 7))) return FVM_ERR_ARG;
        if (a.sh <= 0 || a.sw <= 0 || a.dh <= 0 || a.dw <= 0 || a.ph < 0 || a.pw < 0) return FVM_ERR_ARG;
        if (a.ldx < a.C || a.ldy < a.K || (a.res && a.ldr < a.K)) return FVM_ERR_ARG;
        if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.w) & 15) ||
            (reinterpret_cast<uintptr_t>(a.y) & 15) || (reinterpret_cast<uintptr_t>(a.res) & 15) ||
            (reinterpret_cast<uintptr_t>(a.bias) & 15) || (reinterpret_cast<uintptr_t>(a.scale) & 15))
            return FVM_ERR_ARG;
        if (a.act < 0 || a.act > 6) return FVM_ERR_ARG;
        const int P = (a.H + 2 * a.ph - a.dh * (a.R - 1) - 1) / a.sh + 1;
        const int Q = (a.W + 2 * a.pw - a.dw * (a.S - 1) - 1) / a.sw + 1;
        if (P <= 0 || Q <= 0) return FVM_ERR_ARG;
        const long long M_ll = static_cast<long long>(a.N) * P * Q;
        if (M_ll > 0x3fffff00ll || static_cast<long long>(a.N) * a.H * a.W > 0x3fffff00ll) return FVM_ERR_ARG;
        L.M = static_cast<int>(M_ll);
        L.K = a.K; L.P = P; L.Q = Q; L.H = a.H; L.W = a.W; L.S = a.S;
        L.sh = a.sh; L.sw = a.sw; L.ph = a.ph; L.pw = a.pw; L.dh = a.dh; L.dw = a.dw;
        L.rspan = (a.R - 1) * a.dh;
        L.cchunks = (a.C + BK - 1) / BK;
        L.kblocks = a.R * a.S * L.cchunks;
        int bn = a.tile_n & 0xffff;
        // 128-wide tiles: one cut of the staging region for all layers, three buffers of it, many tiles per layer
        if (bn == 0) bn = a.K <= 128 ? (a.K + 31) / 32 * 32 : 128;
        if (bn < 32 || bn > 256 || (bn & 31)) return FVM_ERR_ARG;
        L.BN = bn;
        L.n_tiles = (a.K + bn - 1) / bn;
        if (L.n_tiles > 1 && (bn & 63)) return FVM_ERR_ARG;
        L.m_tiles = (L.M + 2 * BM - 1) / (2 * BM);
        L.nsub = (bn + 63) / 64;
        L.im2col = !(a.R == 1 && a.S == 1 && a.sh == 1 && a.sw == 1 && a.ph == 0 && a.pw == 0);
        L.act = a.act;
        L.has_res = a.res != nullptr;
        L.bias = static_cast<const __half*>(a.bias);
        L.scale = a.scale;
        L.bias_elems = L.n_tiles * bn;
        L.div_ntiles = fastdiv_init(static_cast<uint32_t>(L.n_tiles));
        L.div_pq = fastdiv_init(static_cast<uint32_t>(P) * Q);
        L.div_q = fastdiv_init(static_cast<uint32_t>(Q));
        L.done_count = 2 * L.n_tiles;
        L.tile0 = tiles;
        L.flag0 = flags;
        const long long lt = static_cast<long long>(L.m_tiles) * L.n_tiles;
        if (tiles + lt > 0x3fffffffll) return FVM_ERR_ARG;
        tiles += static_cast<int>(lt);
        flags += L.m_tiles;
        if (bn > max_bn) max_bn = bn;
        if (L.bias_elems > max_bias) max_bias = L.bias_elems;
        xbytes[i] = (static_cast<size_t>(a.N) * a.H * a.W - 1) * a.ldx * 2 + static_cast<size_t>(a.C) * 2;
        ybytes[i] = (static_cast<size_t>(L.M) - 1) * a.ldy * 2 + static_cast<size_t>(a.K) * 2;
        // producers: the latest earlier layer whose output is exactly this layer's input / residual
        L.in_layer = L.res_layer = -1;
        for (int j = i - 1; j >= 0; --j) {
            const fvm_chain_layer& b = layers[j];
            const ChainLayer& J = cp.L[j];
            if (L.in_layer < 0 && b.y == a.x) {
                if (b.ldy != a.ldx || b.K != a.C || J.P != a.H || J.Q != a.W || b.N != a.N) return FVM_ERR_ARG;
                L.in_layer = j;
            }
            if (a.res && L.res_layer < 0 && b.y == a.res) {
                if (b.ldy != a.ldr || b.K != a.K || J.M != L.M) return FVM_ERR_ARG;
                L.res_layer = j;
            }
        }
        if (a.res && L.res_layer < 0) {
            // a residual from outside the chain (complete before the launch): its own map
            if (n_ext == CHAIN_MAX_EXT_RES) return FVM_ERR_ARG;
            const unsigned long long dims[2] = {static_cast<unsigned long long>(a.K), static_cast<unsigned long long>(L.M)};
            const unsigned long long strides[1] = {static_cast<unsigned long long>(a.ldr) * 2};
            const unsigned box[2] = {64, BM};
            if (encode_tiled_f16(&cp.ext_res[n_ext], a.res, 2, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
            L.res_ext = n_ext++;
        }
        for (int j = 0; j < i; ++j) {
            const fvm_chain_layer& b = layers[j];
            // an input that overlaps an earlier output without being that output; an output that overlaps anything an
            // earlier layer reads or writes, or this layer's own operands
            if (j != L.in_layer && ranges_overlap(a.x, xbytes[i], b.y, ybytes[j])) return FVM_ERR_ARG;
            if (a.res && j != L.res_layer && ranges_overlap(a.res, ybytes[i], b.y, ybytes[j])) return FVM_ERR_ARG;
            if (ranges_overlap(a.y, ybytes[i], b.y, ybytes[j]) || ranges_overlap(a.y, ybytes[i], b.x, xbytes[j]) ||
                (b.res && ranges_overlap(a.y, ybytes[i], b.res, ybytes[j])))
                return FVM_ERR_ARG;
        }
        if (ranges_overlap(a.y, ybytes[i], a.x, xbytes[i])) return FVM_ERR_ARG;
    }
    if (flags > st->chain_flag_count) return FVM_ERR_ARG;
    cp.total_tiles = tiles;
    cp.flags = st->chain_flags;
    cp.status = st->status_dev;
    // shared memory: slots sized for the widest tile of the chain; three staging buffers of the widest tile if four
    // slots still fit beside them, else two, else one
    cp.stage_bytes = A_STAGE_BYTES + static_cast<uint32_t>(max_bn / 2) * BK * 2;
    const uint32_t max_epi = static_cast<uint32_t>((max_bn + 63) / 64) * SUB_BYTES;
    const uint32_t bias_bytes = (static_cast<uint32_t>(max_bias) * 4 + 15u) & ~15u;
    if (bias_bytes > MAX_BIAS_BYTES) return FVM_ERR_ARG;
    const uint32_t fixed = 1024 + 8 * NUM_BARRIERS + MISC_BYTES + bias_bytes;
    const uint32_t total = 227 * 1024;
    int nbuf = 3;
    while (nbuf > 1 && fixed + static_cast<uint32_t>(nbuf) * max_epi + 4 * cp.stage_bytes > total) --nbuf;
    if (fixed + static_cast<uint32_t>(nbuf) * max_epi + 2 * cp.stage_bytes > total) return FVM_ERR_ARG;
    cp.epi_region_bytes = static_cast<uint32_t>(nbuf) * max_epi;
    cp.stages = static_cast<int>((total - fixed - cp.epi_region_bytes) / cp.stage_bytes);
    if (cp.stages > MAX_STAGES) cp.stages = MAX_STAGES;
    const size_t smem = fixed + static_cast<size_t>(cp.stages) * cp.stage_bytes + cp.epi_region_bytes;
    for (int i = 0; i < n; ++i) {
        const fvm_chain_layer& a = layers[i];
        ChainLayer& L = cp.L[i];
        const uint32_t epi_bytes = static_cast<uint32_t>(L.nsub) * SUB_BYTES;
        L.nepi = static_cast<int>(cp.epi_region_bytes / epi_bytes);
        if (L.nepi > MAX_EPI) L.nepi = MAX_EPI;
        {   // output [M, K], row stride ldy: 64-channel x 128-row boxes (also read as the residual of later layers)
            const unsigned long long dims[2] = {static_cast<unsigned long long>(a.K), static_cast<unsigned long long>(L.M)};
            const unsigned long long strides[1] = {static_cast<unsigned long long>(a.ldy) * 2};
            const unsigned box[2] = {64, BM};
            if (encode_tiled_f16(&L.tmap_y, a.y, 2, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
        }
        {   // weights [K][R*S][C]: this CTA's half of an n-tile per load
            const unsigned long long dims[3] = {static_cast<unsigned long long>(a.C), static_cast<unsigned long long>(a.R) * a.S,
                                                static_cast<unsigned long long>(a.K)};
            const unsigned long long strides[2] = {static_cast<unsigned long long>(a.C) * 2,
                                                   static_cast<unsigned long long>(a.R) * a.S * a.C * 2};
            const unsigned box[3] = {BK, 1, static_cast<unsigned>(L.BN / 2)};
            if (encode_tiled_f16(&L.tmap_b, a.w, 3, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
        }
        if (!L.im2col) {
            const unsigned long long dims[2] = {static_cast<unsigned long long>(a.C), static_cast<unsigned long long>(L.M)};
            const unsigned long long strides[1] = {static_cast<unsigned long long>(a.ldx) * 2};
            const unsigned box[2] = {BK, BM};
            if (encode_tiled_f16(&L.tmap_a, a.x, 2, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
        } else {
            const int up_w = a.pw - (a.S - 1) * a.dw, up_h = a.ph - (a.R - 1) * a.dh;
            if (a.pw > 127 || a.ph > 127 || up_w < -128 || up_h < -128 || (a.S - 1) * a.dw > 255 || (a.R - 1) * a.dh > 255)
                return FVM_ERR_ARG;
            cuuint64_t dims[4] = {static_cast<cuuint64_t>(a.C), static_cast<cuuint64_t>(a.W), static_cast<cuuint64_t>(a.H),
                                  static_cast<cuuint64_t>(a.N)};
            cuuint64_t strides[3] = {static_cast<cuuint64_t>(a.ldx) * 2, static_cast<cuuint64_t>(a.W) * a.ldx * 2,
                                     static_cast<cuuint64_t>(a.H) * a.W * a.ldx * 2};
            int lower[2] = {-a.pw, -a.ph};
            int upper[2] = {up_w, up_h};
            cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(a.sw), static_cast<cuuint32_t>(a.sh), 1};
            CUresult r = g_encode_im2col(&L.tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(a.x), dims, strides,
                                         lower, upper, BK, BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return FVM_ERR_TMAP;
            const unsigned long long bytes = static_cast<unsigned long long>(a.N) * a.H * a.W * a.ldx * 2;
            if (g_driver_version <= 13010 && bytes < 131072ull)      // see conv2d_launch
                reinterpret_cast<uint64_t*>(&L.tmap_a)[1] &= ~(1ull << 21);
        }
    }
    if (cudaMemsetAsync(st->chain_flags, 0, static_cast<size_t>(flags) * sizeof(int), stream) != cudaSuccess)
        return FVM_ERR_LAUNCH;
    const int pairs = tiles < st->pair_clusters ? tiles : st->pair_clusters;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    cfg.blockDim = dim3(CONV_THREADS);
    cfg.dynamicSmemBytes = smem < 120 * 1024 ? 120 * 1024 : smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 2;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, conv_chain_kernel, cp) != cudaSuccess) {
        (void)cudaGetLastError();
        return FVM_ERR_LAUNCH;
    }
    count_launch();
    return FVM_OK;
}


// ------------------------------------------------------------------------------------------------ two layers, one launch
// y = act1(x * w1^T + b1 [+ res]) ([M, K1], row stride ldy) and z = act2(y * w2^T + b2) ([M, K2], row stride ldz) as one
// launch of conv_dual_kernel. x [M, C1] (row stride ldx), w1 [K1][C1], w2 [K2][K1]; (C1, K1) is (64, 128), (64, 256) or
// (128, 128), K2 a multiple of 16 up to 128; activations 0 (none) or 1 (ReLU) run specialised, the others through the generic code.
// Refused (FVM_ERR_ARG, nothing launched): other shapes, misaligned pointers, outputs that overlap an input or each other.
int conv_dual_launch(const void* x, const void* w1, const void* b1, const void* res, void* y, const void* w2, const void* b2,
                     void* z, long long M, int C1, int K1, int K2, long long ldx, long long ldr, long long ldy, long long ldz,
                     int act1, int act2, cudaStream_t stream) {
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    if (!x || !w1 || !y || !w2 || !z) return FVM_ERR_ARG;
    if (M <= 0 || M > 0x7fffff00ll) return FVM_ERR_ARG;
    if ((C1 != 64 && C1 != 128) || (K1 != 128 && K1 != 256) || C1 * K1 > 64 * 256 || K2 < 16 || K2 > 128 || (K2 & 15)) return FVM_ERR_ARG;
    if (act1 < 0 || act1 > 6 || act2 < 0 || act2 > 6) return FVM_ERR_ARG;
    if ((ldx & 7) || ldx < C1 || (ldy & 7) || ldy < K1 || (ldz & 7) || ldz < K2 || (res && ((ldr & 7) || ldr < K1))) return FVM_ERR_ARG;
    const void* ptrs[8] = {x, w1, b1, res, y, w2, b2, z};
    for (int i = 0; i < 8; ++i)
        if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15) return FVM_ERR_ARG;
    {
        const size_t nx = static_cast<size_t>((M - 1) * ldx + C1) * 2, ny = static_cast<size_t>((M - 1) * ldy + K1) * 2;
        const size_t nz = static_cast<size_t>((M - 1) * ldz + K2) * 2, nr = res ? static_cast<size_t>((M - 1) * ldr + K1) * 2 : 0;
        if (ranges_overlap(y, ny, x, nx) || ranges_overlap(z, nz, x, nx) || ranges_overlap(y, ny, z, nz)) return FVM_ERR_ARG;
        if (res && (ranges_overlap(y, ny, res, nr) || ranges_overlap(z, nz, res, nr))) return FVM_ERR_ARG;
    }
    DualParams p;
    memset(&p, 0, sizeof(p));
    p.M = static_cast<int>(M);
    p.m_tiles = static_cast<int>((M + BM - 1) / BM);
    p.kb1 = C1 / 64;
    p.K1 = K1;
    p.N2 = K2;
    // z up to 64 channels: y in units of 128 channels, three slots (3 x 128 + 2 x 64 TMEM columns); wider z: units of 64
    // channels, four slots (4 x 64 + 2 x 128 columns) -- shared memory then still holds both weight tensors
    p.UW = K2 <= 64 ? 128 : 64;
    p.UP = p.UW / 64;
    p.ys = K2 <= 64 ? 3 : 4;
    p.H = K1 / p.UW;
    p.acc2_col = p.ys * p.UW;
    p.acc2_stride = K2 <= 64 ? 64 : 128;
    p.zp = (K2 + 63) / 64;
    p.act1 = act1;
    p.act2 = act2;
    p.has_res = res != nullptr;
    p.bias1 = static_cast<const __half*>(b1);
    p.bias2 = static_cast<const __half*>(b2);
    p.status = st->status_dev;
    {
        // x and the identity are dead after this launch in a bottleneck block (evict-first, as for a single layer with a
        // residual in conv2d_launch); z is what the very next layer reads: kept. Keeping y (the next identity, read one
        // layer later) as well or instead measured the same or slightly slower inside a ResNet-50 forward.
        static const int use_hints = [] { const char* v = getenv("FVM_B200_L2_HINTS"); return (v && v[0] == '0') ? 0 : 1; }();
        if (use_hints && res) {
            p.hints = 1 | 2;
            if (static_cast<unsigned long long>(M) * K2 * 2 <= 112ull * 1024 * 1024) p.hints |= 8;
        }
    }
    const uint32_t fixed = 1024 + static_cast<uint32_t>(p.kb1 * K1) * 128u + static_cast<uint32_t>((K1 / 64) * K2) * 128u +
                           static_cast<uint32_t>(p.ys * p.UP + p.zp) * SUB_BYTES + 8 * DUAL_NUM_BARRIERS + DUAL_MISC_BYTES +
                           ((static_cast<uint32_t>(K1 + K2) * 4 + 15u) & ~15u);
    const uint32_t a_stage = static_cast<uint32_t>(p.kb1) * A_STAGE_BYTES;
    if (fixed + 2 * a_stage > 227u * 1024) return FVM_ERR_ARG;
    p.sa = static_cast<int>((227u * 1024 - fixed) / a_stage);
    if (p.sa > DUAL_MAX_SA) p.sa = DUAL_MAX_SA;
    size_t smem = fixed + static_cast<size_t>(p.sa) * a_stage;
    if (smem < 120 * 1024) smem = 120 * 1024;          // one CTA per SM: it owns all 512 TMEM columns

    CUtensorMap tmap_a, tmap_w1, tmap_r, tmap_y, tmap_w2, tmap_z;
    const unsigned long long Mu = static_cast<unsigned long long>(M);
    {
        const unsigned long long dims[2] = {static_cast<unsigned long long>(C1), Mu};
        const unsigned long long strides[1] = {static_cast<unsigned long long>(ldx) * 2};
        const unsigned box[2] = {BK, BM};
        if (encode_tiled_f16(&tmap_a, x, 2, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
    }
    {
        const unsigned long long dims[2] = {static_cast<unsigned long long>(K1), Mu};
        const unsigned long long ystr[1] = {static_cast<unsigned long long>(ldy) * 2};
        const unsigned box[2] = {64, BM};
        if (encode_tiled_f16(&tmap_y, y, 2, dims, ystr, box, true) != FVM_OK) return FVM_ERR_TMAP;
        if (res) {
            const unsigned long long rstr[1] = {static_cast<unsigned long long>(ldr) * 2};
            if (encode_tiled_f16(&tmap_r, res, 2, dims, rstr, box, true) != FVM_OK) return FVM_ERR_TMAP;
        } else {
            tmap_r = tmap_y;
        }
    }
    {
        const unsigned long long dims[2] = {static_cast<unsigned long long>(K2), Mu};
        const unsigned long long zstr[1] = {static_cast<unsigned long long>(ldz) * 2};
        const unsigned box[2] = {64, BM};
        if (encode_tiled_f16(&tmap_z, z, 2, dims, zstr, box, true) != FVM_OK) return FVM_ERR_TMAP;
    }
    {
        const unsigned long long dims[3] = {static_cast<unsigned long long>(C1), 1ull, static_cast<unsigned long long>(K1)};
        const unsigned long long strides[2] = {static_cast<unsigned long long>(C1) * 2, static_cast<unsigned long long>(C1) * 2};
        const unsigned box[3] = {BK, 1, 128};
        if (encode_tiled_f16(&tmap_w1, w1, 3, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
    }
    {
        const unsigned long long dims[3] = {static_cast<unsigned long long>(K1), 1ull, static_cast<unsigned long long>(K2)};
        const unsigned long long strides[2] = {static_cast<unsigned long long>(K1) * 2, static_cast<unsigned long long>(K1) * 2};
        const unsigned box[3] = {BK, 1, static_cast<unsigned>(K2)};
        if (encode_tiled_f16(&tmap_w2, w2, 3, dims, strides, box, true) != FVM_OK) return FVM_ERR_TMAP;
    }
    const int grid = p.m_tiles < st->sms ? p.m_tiles : st->sms;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(CONV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    static const int use_pdl = [] { const char* v = getenv("FVM_B200_PDL"); return (v && v[0] == '0') ? 0 : 1; }();
    cfg.attrs = attrs;
    cfg.numAttrs = use_pdl ? 1u : 0u;
    if (cudaLaunchKernelEx(&cfg, conv_dual_kernel, tmap_a, tmap_w1, tmap_r, tmap_y, tmap_w2, tmap_z, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return FVM_ERR_LAUNCH;
    }
    count_launch();
    return FVM_OK;
}

}  // namespace fvm
