// Library state and the C-ABI entry points that are not tied to one kernel file.
#include <atomic>
#include <mutex>

#include "fvm_internal.h"
#include "ptx_sm100.cuh"

namespace fvm {

static constexpr int MAX_DEVICES = 64;
static DeviceState g_state[MAX_DEVICES];
static std::mutex g_mutex;
static std::atomic<long long> g_launches{0};

DeviceState* device_state() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    DeviceState* st = &g_state[dev];
    return st->ready ? st : nullptr;
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// Self-test of the bounded-wait path every kernel role relies on: one thread waits on an mbarrier that nothing ever
// arrives at, with a limit of `limit_ns`; the wait gives up, the status word receives 0x1ff and the kernel returns by
// itself. No trap, no unbounded spin: the context stays usable.
static constexpr int STATUS_SELFTEST_WAIT = 0x1ff;
__global__ void wait_expiry_kernel(int* status, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait<32>(smem_u32(&bar), 0u, &abort_flag, limit_ns)) atomicExch(status, STATUS_SELFTEST_WAIT);
}

}  // namespace fvm

using namespace fvm;

extern "C" int fvm_selftest_wait_expiry(int limit_us, void* stream) {
    DeviceState* st = device_state();
    if (!st) return FVM_ERR_SETUP;
    if (limit_us <= 0 || limit_us > 100000) return FVM_ERR_ARG;      // at most 0.1 s
    wait_expiry_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st->status_dev,
                                                                        static_cast<unsigned long long>(limit_us) * 1000ull);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? FVM_OK : FVM_ERR_LAUNCH;
}

extern "C" int fvm_init(void) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return FVM_ERR_SETUP;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* st = &g_state[dev];
    if (st->ready) return FVM_OK;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return FVM_ERR_SETUP;
    if (prop.major != 10) return FVM_ERR_SETUP;   // tcgen05 / TMEM kernels: sm_100 family only
    st->sms = prop.multiProcessorCount;
    st->max_smem = static_cast<int>(prop.sharedMemPerBlockOptin);
    // The status word lives in mapped pinned host memory: kernels write it through the device alias, the host reads
    // it after a synchronise without a copy.
    if (cudaHostAlloc(reinterpret_cast<void**>(&st->status_host), sizeof(int), cudaHostAllocMapped) != cudaSuccess)
        return FVM_ERR_SETUP;
    *st->status_host = 0;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&st->status_dev), st->status_host, 0) != cudaSuccess)
        return FVM_ERR_SETUP;
    const int rc = conv_host_init();
    if (rc != FVM_OK) return rc;
    // stream-K scratch: one [128][256] fp32 slot and one counter per SM (19 MB on a 148-SM part). Without it the
    // convolution simply never chooses its stream-K variant.
    {
        const size_t floats = static_cast<size_t>(st->sms) * 128 * 256;
        if (cudaMalloc(reinterpret_cast<void**>(&st->sk_part), floats * sizeof(float)) == cudaSuccess &&
            cudaMalloc(reinterpret_cast<void**>(&st->sk_flags), static_cast<size_t>(st->sms) * sizeof(int)) == cudaSuccess &&
            cudaMemset(st->sk_flags, 0, static_cast<size_t>(st->sms) * sizeof(int)) == cudaSuccess) {
            st->sk_floats = floats;
        } else {
            (void)cudaGetLastError();
            st->sk_part = nullptr;
            st->sk_floats = 0;
        }
    }
    st->pair_clusters = conv_pair_capacity();
    {
        const int count = 1 << 16;
        if (cudaMalloc(reinterpret_cast<void**>(&st->chain_flags), static_cast<size_t>(count) * sizeof(int)) == cudaSuccess) {
            st->chain_flag_count = count;
        } else {
            (void)cudaGetLastError();
            st->chain_flags = nullptr;
        }
    }
    st->ready = true;
    return FVM_OK;
}

extern "C" long long fvm_query(int what) {
    DeviceState* st = device_state();
    switch (what) {
        case 0: return 100;   // version 0.1.0
        case 1: return st ? st->sms : -1;
        case 2: return st ? st->max_smem : -1;
        case 3: return g_launches.load(std::memory_order_relaxed);
        case 4: return st ? st->pair_clusters : -1;   // CTA pairs resident at once (0: pair kernel unavailable)
    }
    return -1;
}

extern "C" int fvm_last_status(int* code) {
    DeviceState* st = device_state();
    if (!st || !code) return FVM_ERR_SETUP;
    *code = *static_cast<volatile int*>(st->status_host);
    *static_cast<volatile int*>(st->status_host) = 0;
    // a kernel that gave up may have left stream-K counters raised: clear them so that later launches start clean
    if (*code != 0 && st->sk_flags) cudaMemset(st->sk_flags, 0, static_cast<size_t>(st->sms) * sizeof(int));
    return FVM_OK;
}

extern "C" int fvm_conv_chain_f16(const fvm_chain_layer* layers, int n_layers, void* stream) {
    return conv_chain_launch(layers, n_layers, static_cast<cudaStream_t>(stream));
}

extern "C" int fvm_conv_dual_f16(const void* x, const void* w1, const void* b1, const void* res, void* y, const void* w2,
                                 const void* b2, void* z, long long M, int C1, int K1, int K2, long long ldx, long long ldr,
                                 long long ldy, long long ldz, int act1, int act2, void* stream) {
    return conv_dual_launch(x, w1, b1, res, y, w2, b2, z, M, C1, K1, K2, ldx, ldr, ldy, ldz, act1, act2,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int fvm_conv2d_f16(const void* x, const void* w, const void* bias, const void* res, const float* scale,
                              void* y, int N, int H, int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw,
                              int dh, int dw, long long ldx, long long ldy, long long ldr, int act, void* stream) {
    return conv2d_launch(x, w, bias, res, scale, y, N, H, W, C, K, R, S, ph, pw, sh, sw, dh, dw, ldx, ldy, ldr, act, 0, -1,
                         -1, static_cast<cudaStream_t>(stream));
}

// Same as fvm_conv2d_f16 with the tile shape forced: tile_n low 16 bits = output-channel tile (multiple of 32, <= 256;
// 0 = choose), bits 16 and up = 128-pixel sub-tiles per tile (1, 2 or 4; 0 = choose). Used by tests and by the host's
// per-layer tuning to exercise every tile shape on one problem.
extern "C" int fvm_conv2d_f16_tile(const void* x, const void* w, const void* bias, const void* res, const float* scale,
                                   void* y, int N, int H, int W, int C, int K, int R, int S, int ph, int pw, int sh,
                                   int sw, int dh, int dw, long long ldx, long long ldy, long long ldr, int act,
                                   int tile_n, void* stream) {
    return conv2d_launch(x, w, bias, res, scale, y, N, H, W, C, K, R, S, ph, pw, sh, sw, dh, dw, ldx, ldy, ldr, act,
                         tile_n, -1, -1, static_cast<cudaStream_t>(stream));
}

// fvm_conv2d_f16_tile with separate bottom / right padding (ph_hi, pw_hi; negative = same as top / left): used by the
// host when it re-expresses a stride-2 RGB stem over column pairs (16 channels per tap), where the two sides differ.
extern "C" int fvm_conv2d_f16_pad(const void* x, const void* w, const void* bias, const void* res, const float* scale,
                                  void* y, int N, int H, int W, int C, int K, int R, int S, int ph, int pw, int sh,
                                  int sw, int dh, int dw, long long ldx, long long ldy, long long ldr, int act,
                                  int tile_n, int ph_hi, int pw_hi, void* stream) {
    return conv2d_launch(x, w, bias, res, scale, y, N, H, W, C, K, R, S, ph, pw, sh, sw, dh, dw, ldx, ldy, ldr, act,
                         tile_n, ph_hi, pw_hi, static_cast<cudaStream_t>(stream));
}

// Grouped convolution on the dense kernel: see fvm_gconv2d_f16 in the header.
extern "C" int fvm_gconv2d_f16(const void* x, const void* w_sg, const void* bias, const void* res, void* y, int N, int H,
                               int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                               long long ldx, long long ldy, long long ldr, int act, int gsg, int gsk, void* stream) {
    if (gsg <= 0) return FVM_ERR_ARG;
    return conv2d_launch(x, w_sg, bias, res, nullptr, y, N, H, W, C, K, R, S, ph, pw, sh, sw, dh, dw, ldx, ldy, ldr, act, 0,
                         -1, -1, static_cast<cudaStream_t>(stream), 0, gsg, gsk);
}

// 1x1 stride-1 convolution whose weights differ per image: w_n is [N][K][C]. Used for the project conv of a
// squeeze-excite block with the gate folded into the weights (see fvm_gate_weights_f16).
extern "C" int fvm_conv1x1_wbatch_f16(const void* x, const void* w_n, const void* bias, const void* res, void* y, int N,
                                      int H, int W, int C, int K, long long ldx, long long ldy, long long ldr, int act,
                                      void* stream) {
    return conv2d_launch(x, w_n, bias, res, nullptr, y, N, H, W, C, K, 1, 1, 0, 0, 1, 1, 1, 1, ldx, ldy, ldr, act, 0, -1, -1,
                         static_cast<cudaStream_t>(stream), 1);
}

// Stride-2 stem on the column-parity-split 8-channel input (see stem_s2_launch).
extern "C" int fvm_stem_conv_s2_f16(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int K,
                                    int R, int S, int ph, int pw, long long ldy, int act, void* stream) {
    return stem_s2_launch(x, w, bias, y, N, H, W, K, R, S, ph, pw, ldy, act, static_cast<cudaStream_t>(stream));
}
