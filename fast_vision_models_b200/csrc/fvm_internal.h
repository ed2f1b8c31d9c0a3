// Internal declarations shared by the translation units of libfvm_b200 (not part of the C ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/fvm_b200.h"

namespace fvm {

struct DeviceState {
    int sms = 0;
    int max_smem = 0;
    int* status_dev = nullptr;    // device-visible address of the status word (mapped pinned host memory)
    int* status_host = nullptr;   // host address of the same word
    // stream-K scratch of the convolution kernel: fp32 partial tiles (one slot per CTA) and one counter per slot. Shared
    // by every stream of the device: stream-K launches on different streams must not overlap in time.
    float* sk_part = nullptr;
    int* sk_flags = nullptr;
    size_t sk_floats = 0;
    // completion counters of the layer-chain kernel (one per layer and 256-row tile), zeroed before every chain launch;
    // shared by every stream of the device: chain launches on different streams must not overlap in time
    int* chain_flags = nullptr;
    int chain_flag_count = 0;
    int pair_clusters = 0;        // CTA pairs (clusters of two) the device runs at once; 0: pair kernel unavailable
    bool ready = false;
};

// State of the current device, or nullptr if fvm_init() has not run for it.
DeviceState* device_state();
void count_launch();

int conv_host_init();
int conv_pair_capacity();
// cuTensorMapEncodeTiled for an fp16 tensor of `rank` dimensions (innermost first): sizes, byte strides of dimensions
// 1.., box; no interleave, 128-byte swizzle or none, zero fill outside the tensor. Returns an FVM_* status.
int encode_tiled_f16(CUtensorMap* map, const void* ptr, int rank, const unsigned long long* dims,
                     const unsigned long long* strides_bytes, const unsigned* box, bool swizzle128);
int stem_s2_launch(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int K, int R, int S,
                   int ph, int pw, long long ldy, int act, cudaStream_t stream);
int conv2d_launch(const void* x, const void* w, const void* bias, const void* res, const float* scale, void* y, int N,
                  int H, int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                  long long ldx, long long ldy, long long ldr, int act, int force_bn, int ph_hi, int pw_hi,
                  cudaStream_t stream, int w_per_image = 0, int gsg = 0, int gsk = 0);
int conv_chain_launch(const fvm_chain_layer* layers, int n, cudaStream_t stream);
int conv_dual_launch(const void* x, const void* w1, const void* b1, const void* res, void* y, const void* w2, const void* b2,
                     void* z, long long M, int C1, int K1, int K2, long long ldx, long long ldr, long long ldy, long long ldz,
                     int act1, int act2, cudaStream_t stream);

}  // namespace fvm
