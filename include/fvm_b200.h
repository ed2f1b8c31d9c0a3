/* fvm_b200 -- C ABI of the B200 (sm_100a) convolutional hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, i.e. a cudaStream_t),
 * launches asynchronously on that stream and returns an int status at once:
 *   0 ok, 1 bad argument / unsupported shape, 2 attribute or set-up failure, 3 launch error, 4 tensor-map encode error.
 * The same convention as the reference's `run<F>` (classification/fast/csrc/fused_conv.cu:152-173: 0 ok, 1 cannot
 * implement, 2 shared-memory attribute failed, 3 launch error). Asynchronous faults (a bounded device-side wait that
 * ran out) are written to a per-device status word that fvm_last_status() reads after the stream has been synchronised.
 *
 * Tensors: activations are NHWC fp16 (a channels-last NCHW tensor in torch terms); `ld*` arguments are the pixel
 * stride in elements (>= channels; a channel slice of a wider buffer is allowed, as in the reference's `ldx`/`ldy`,
 * fused_conv.cu:24-31). Dense weights are KRSC fp16, depthwise weights RSC fp16, bias fp16 [K]. Base pointers and pixel
 * strides must be 16-byte aligned (channels % 8 == 0), which is the reference's own contract (fused_conv.cu:7).
 *
 * Nothing here allocates device memory per call; fvm_init() sets up the per-device state and must be called once per
 * device before the first launch (and before any stream capture).
 */
#ifndef FVM_B200_H
#define FVM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FVM_OK 0
#define FVM_ERR_ARG 1
#define FVM_ERR_SETUP 2
#define FVM_ERR_LAUNCH 3
#define FVM_ERR_TMAP 4

/* activation codes: reference act_f, classification/fast/csrc/fused_conv.cu:33-43 */
#define FVM_ACT_NONE 0
#define FVM_ACT_RELU 1
#define FVM_ACT_RELU6 2
#define FVM_ACT_SILU 3
#define FVM_ACT_HARDSWISH 4
#define FVM_ACT_GELU_ERF 5
#define FVM_ACT_GELU_TANH 6

/* Per-device set-up for the current device (SM count, kernel attributes, status word). Idempotent.
 * Replaces the static initialisers of the reference extensions (fused_conv.cu:165-170, :205). */
int fvm_init(void);

/* what: 0 library version, 1 SM count of the current device, 2 max dynamic shared memory per block (bytes),
 * 3 number of kernels launched by this library since load (all devices), 4 number of two-CTA clusters the current
 * device runs at once (0: the CTA-pair convolution kernel is unavailable). */
long long fvm_query(int what);

/* Reads and clears the asynchronous status word of the current device (0 = no fault). Call after synchronising. */
int fvm_last_status(int* code);

/* Self-test of the fault path -- no counterpart in the reference (its kernels have no device-side waits). Launches one
 * small kernel whose only thread waits, for at most limit_us microseconds (1..100000), on a barrier that nothing arrives
 * at; the wait runs out, the kernel writes 0x1ff to the status word and returns. After a synchronise fvm_last_status
 * reports 0x1ff and the device is as usable as before. */
int fvm_selftest_wait_expiry(int limit_us, void* stream);

/* Dense convolution / GEMM with fused epilogue -- replaces clf::conv_fused / conv_fused_into
 * (classification/fast/csrc/fused_conv.cu:231-306), segx::conv_fused_d (segmentation/fast/csrc/segx_conv.cu:231-299)
 * and clfr3::pw (classification/fast/csrc/r3.cu:633-765):
 *   y[n,p,q,k] = act( (sum_{r,s,c} x[n, p*sh-ph+r*dh, q*sw-pw+s*dw, c] * w[k,r,s,c] + bias[k]) * scale[k] + res[n,p,q,k] )
 * fp16 operands, fp32 accumulation (TMEM), fp32 epilogue, one rounding to fp16. bias, scale (fp32 [K], a LayerScale
 * that was not folded into w) and res may be NULL. Requires C % 8 == 0 and K % 8 == 0; x, w, y, res, bias AND scale
 * must be 16-byte aligned (scale is read as float4): a misaligned pointer returns 1 before anything is launched. */
int fvm_conv2d_f16(const void* x, const void* w, const void* bias, const void* res, const float* scale, void* y,
                   int N, int H, int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                   long long ldx, long long ldy, long long ldr, int act, void* stream);

/* fvm_conv2d_f16 with the tile shape forced -- the counterpart of the reference's `cfg` argument of clf::conv_fused
 * (fused_conv.cu:180-227, a tile-configuration index). tile_n: low 16 bits = output-channel tile (multiple of 32, at
 * most 256; 0 = choose), bits 16..23 = 128-pixel sub-tiles per tile (1, 2, 4; 0 = choose), bits 24..25 = keep the
 * weight tile resident in shared memory (0 = choose, 1 = on, 2 = off), bits 26..27 = halo mode, same coding: a 3x3
 * stride-1 convolution (dilation 1..4) walks 16 x 8 patches of output pixels and reads each patch's input (with its
 * border) once per 64 channels instead of once per filter tap; bits 28..29 = stream-K, same coding: the k-blocks of all
 * tiles are cut into one equal run per SM (for layers with fewer tiles than SMs); tiles whose k-blocks fall into
 * several runs are summed in fp32 through a per-device scratch buffer that all streams share, so two stream-K launches
 * on different streams of one device must not overlap in time; bit 30 = CTA pairs: two CTAs on neighbouring SMs (a
 * cluster of two) share each tile of 256 pixels x tile_n channels through tcgen05.mma.cta_group::2 and each loads only
 * half of the weight tile (for layers bound by re-reading the weights from L2; same results as the single-CTA kernel
 * bit for bit; not with sub-tiles, halo, weight-resident or stream-K mode). Shapes that do not fit return 1. */
int fvm_conv2d_f16_tile(const void* x, const void* w, const void* bias, const void* res, const float* scale, void* y,
                        int N, int H, int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                        long long ldx, long long ldy, long long ldr, int act, int tile_n, void* stream);

/* Grouped convolution -- replaces clfr3::gconv2 (classification/fast/csrc/r3.cu:49-299; a hand-written grouped
 * implicit GEMM there) and, with a group width of one, clfmb::dwmult (depthwise with channel multiplier). It runs on the
 * dense tcgen05 kernel as block-diagonal convolutions over "super-groups": the channels are cut into runs of gsg input
 * and gsk output channels that hold whole groups (gsg a multiple of the group width and of 8, gsk = gsg * K / C a
 * multiple of 64 unless one run covers everything; the last run may be short), and w_sg is [K][R][S][gsg] with each
 * output channel's own group's weights in place and zeros elsewhere (fast_vision_models_b200.fold.pack_grouped builds it
 * from the reference's [K][GW][R][S] weights). An output tile reads only its run's input channels, so the work grows
 * with gsg / GW, not with the number of groups. Same epilogue as fvm_conv2d_f16 (bias, residual, activation). */
int fvm_gconv2d_f16(const void* x, const void* w_sg, const void* bias, const void* res, void* y, int N, int H, int W, int C,
                    int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw, long long ldx, long long ldy,
                    long long ldr, int act, int gsg, int gsk, void* stream);

/* A run of dense convolutions as ONE launch -- no counterpart in the reference, which launches one kernel per layer
 * (classification/fast/csrc/fused_conv.cu:231-306): the bottleneck blocks of a ResNet stage, say. Each entry is one
 * fvm_conv2d_f16 call (same operands, same arithmetic, same bits as the CTA-pair kernel of fvm_conv2d_f16_tile); layer
 * i may read, as input or residual, the output of an earlier entry (recognised by pointer, shape and row stride), and
 * its tiles start as soon as the tiles that hold those pixels are complete, so consecutive layers overlap instead of
 * paying a launch, a pipeline start and a partial last wave each. Everything else a layer reads must be complete
 * before the call (stream order). Returns 1 with nothing launched when the chain cannot be expressed: more than 48
 * layers, fewer than 24 input channels, more than 4 residuals that no entry produces, or buffers that alias one another
 * (an output that overlaps any other operand of the chain; layers do not run in stream order). tile_n: output-channel tile
 * (0 = choose). Chain launches on different streams of one device must not overlap in time (shared counters). */
typedef struct fvm_chain_layer {
    const void* x;
    const void* w;
    const void* bias;
    const void* res;
    const float* scale;
    void* y;
    int N, H, W, C, K, R, S, ph, pw, sh, sw, dh, dw;
    long long ldx, ldy, ldr;
    int act;
    int tile_n;
} fvm_chain_layer;
int fvm_conv_chain_f16(const fvm_chain_layer* layers, int n_layers, void* stream);

/* Two 1x1 convolutions as ONE launch, the first layer's output handed to the second on chip -- no counterpart in the
 * reference (one kernel per layer, classification/fast/csrc/fused_conv.cu:231-306); it takes the last convolution of a
 * bottleneck block and the first of the next (torchvision Bottleneck.conv3 -> add -> ReLU -> next Bottleneck.conv1):
 *   y = act1(x * w1^T + b1 [+ res])   x [M, C1] (row stride ldx), w1 [K1][C1], res / y [M, K1] (row strides ldr / ldy)
 *   z = act2(y * w2^T + b2)           w2 [K2][K1], z [M, K2] (row stride ldz)
 * y is written to global memory once and read by the second layer from the shared-memory tile it was stored from, so
 * the second layer costs its weights and its output only. Same bits as two fvm_conv2d_f16 calls. (C1, K1) is (64, 128),
 * (64, 256) or (128, 128) (both weight tensors stay in shared memory), K2 a multiple of 16 up to 128; returns 1 with
 * nothing launched for other shapes, for misaligned pointers (16 bytes) or when y or z overlaps another operand. */
int fvm_conv_dual_f16(const void* x, const void* w1, const void* b1, const void* res, void* y, const void* w2,
                      const void* b2, void* z, long long M, int C1, int K1, int K2, long long ldx, long long ldr,
                      long long ldy, long long ldz, int act1, int act2, void* stream);

/* fvm_conv2d_f16_tile with separate bottom / right padding (ph_hi, pw_hi; negative = same as top / left). The host
 * uses it to run a stride-2 RGB stem (reference: the zero-padded 8-channel stem, fused.py:90-105) over column pairs:
 * the NHWC8 input viewed as [N, H, W/2, 16] with re-packed weights, which halves the rows the TMA unit gathers. */
int fvm_conv2d_f16_pad(const void* x, const void* w, const void* bias, const void* res, const float* scale, void* y,
                       int N, int H, int W, int C, int K, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw,
                       long long ldx, long long ldy, long long ldr, int act, int tile_n, int ph_hi, int pw_hi,
                       void* stream);

/* Depthwise RxS convolution -- replaces clf::dwconv (fused_conv.cu:418-502), clfr3::dwconv2 (r3.cu:335-454) and
 * segx::dwconv (segmentation/fast/seg_kernels.cu:124-158):
 *   y[n,p,q,c] = act( bias[c] + sum_{r,s} x[n, p*sh-ph+r*dh, q*sw-pw+s*dw, c] * w[r,s,c] )
 * Square 3/5/7-tap filters with stride 1 or 2 and no dilation use the arithmetic of dwconv2 (fp16x2 FMAs within a
 * kernel row, fp32 across rows); every other shape accumulates in fp32 throughout.
 * Fused squeeze (cf. gconv2_pool, r3.cu:181-203): if pool_partial != NULL it receives fp32 partial sums of the
 * fp16-rounded outputs, laid out [N][slots][C] with slots = fvm_dwconv_pool_slots(...) for the same geometry; every
 * element is written (no zeroing needed) and the sums do not depend on scheduling (no atomics). The mean over the
 * pixels is sum over slots / (P*Q): fvm_se_gate_pooled_f16 takes the partial sums as they are. */
int fvm_dwconv_pool_slots(int N, int H, int W, int C, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw);
int fvm_dwconv_f16(const void* x, const void* w_rsc, const void* bias, void* y, float* pool_partial, int N, int H, int W,
                   int C, int R, int S, int ph, int pw, int sh, int sw, int dh, int dw, long long ldx, long long ldy,
                   int act, void* stream);

/* NHWC max / average pooling -- replaces clf::maxpool (fused_conv.cu:338-374) and clf::avgpool (:556-594).
 * P, Q are the output sizes (the caller applies the floor / ceil rule of fused_conv.cu:363-367). */
int fvm_maxpool_f16(const void* x, void* y, int N, int H, int W, int C, int kh, int kw, int sh, int sw, int ph, int pw,
                    int P, int Q, void* stream);
int fvm_avgpool_f16(const void* x, void* y, int N, int H, int W, int C, int kh, int kw, int sh, int sw, int ph, int pw,
                    int P, int Q, int count_include_pad, void* stream);

/* Global average pool, NHWC fp16 [N,HW,C] (pixel stride ldx) -> fp16 [N,C], fp32 accumulation in a fixed order
 * (deterministic). Stands where the reference leaves aten AdaptiveAvgPool2d(1) in the graph
 * (classification/fast/r3.py:188-199) or fuses sums with atomics (r3.cu:181-203, :283-286).
 * `partial` is caller-provided fp32 scratch of at least fvm_gap_scratch_floats(N, HW, C) floats. */
long long fvm_gap_scratch_floats(int N, int HW, int C);
int fvm_global_avgpool_f16(const void* x, void* y, float* partial, int N, int HW, int C, long long ldx, void* stream);

/* Allocation-free variant of fvm_global_avgpool_f16 -- no counterpart in the reference. For callers that cannot
 * obtain device memory at call time: code that runs while a stream is being captured, a serving loop that must never
 * enter the driver's allocator, or a host process whose memory was carved up once at start-up and has no scratch to
 * lend. The partial sums live in a 4 MiB array that is part of the library image on every GPU that loads it, so the
 * caller passes only input and output. Returns 1 (FVM_ERR_ARG) when the problem needs more than
 * fvm_global_avgpool_f16_noalloc_max_floats() floats of scratch (N * splits * C, the value fvm_gap_scratch_floats
 * reports) -- it never falls back to allocating. The first call on a device looks up the array's device address (no
 * allocation); make that call before any stream capture. All calls on a device share the one array: two calls whose
 * kernels can overlap on the GPU (different streams, no ordering) race on it; calls ordered on one stream do not.
 * Nothing in the array has to be cleared between calls. Results are bit-identical to fvm_global_avgpool_f16. */
long long fvm_global_avgpool_f16_noalloc_max_floats(void);
int fvm_global_avgpool_f16_noalloc(const void* x, void* y, int N, int HW, int C, long long ldx, void* stream);

/* Squeeze-excite gate: s[n,:] = W2 * act(W1 * g[n,:] + b1) + b2 with g fp16 [N,C], W1 fp16 [Cs,C], W2 fp16 [C,Cs];
 * stands for the two clf::conv_fused calls on [N,C,1,1] tensors the reference issues (r3.py:188-199). Output fp16 [N,C]
 * (pre-sigmoid). If mean_scale != 0, g is read as fp32 sums [N,C] and multiplied by mean_scale first (fused squeeze). */
int fvm_se_gate_f16(const void* g, const void* w1, const void* b1, const void* w2, const void* b2, void* s, int N,
                    int C, int Cs, int act, float mean_scale, void* stream);

/* The same gate fed by the fused squeeze of fvm_dwconv_f16: `partial` is fp32 [N][slots][C]; g[n,c] =
 * half(mean_scale * sum over slots), slots added in order (deterministic). Replaces the pair gconv2_pool +
 * sums_to_mean_k of the reference (r3.cu:181-203, :283-299), which accumulates with atomics. */
int fvm_se_gate_pooled_f16(const float* partial, int slots, const void* w1, const void* b1, const void* w2,
                           const void* b2, void* s, int N, int C, int Cs, int act, float mean_scale, void* stream);

/* The squeeze-excite scale without its pass over the tensor -- no counterpart in the reference, which always runs
 * clfr3::se_scale (r3.cu:302-329) and then the project conv. fvm_gate_weights_f16 folds the rounded gate into the 1x1
 * weights of the conv that follows, per image: out[n][k][c] = half(w[k][c] * half(sigmoid(s[n][c]))), w fp16 [K][C],
 * s fp16 [N][C] (pre-sigmoid), out fp16 [N][K][C]. fvm_conv1x1_wbatch_f16 is the 1x1 stride-1 convolution with such
 * per-image weights: y[n,p,k] = act(sum_c x[n,p,c] * w_n[n][k][c] + bias[k] + res[n,p,k]); an output tile never
 * straddles two images. Same products as scale-then-convolve, the one fp16 rounding of each product's gate factor
 * falls on the weight instead of the activation. */
int fvm_gate_weights_f16(const void* w, const void* s, void* out, int N, int K, int C, void* stream);
int fvm_conv1x1_wbatch_f16(const void* x, const void* w_n, const void* bias, const void* res, void* y, int N, int H, int W,
                           int C, int K, long long ldx, long long ldy, long long ldr, int act, void* stream);

/* y = x * sigmoid(s[n,c]) -- replaces clfr3::se_scale (r3.cu:302-329): sigmoid in fp32, rounded to fp16, fp16 multiply. */
int fvm_se_scale_f16(const void* x, const void* s, void* y, int N, int HW, int C, void* stream);

/* Channels-last LayerNorm over the last dimension of [rows, C] fp16 (row stride ldx / ldy), fp32 two-pass statistics,
 * fp32 affine, one rounding -- the torch nn.LayerNorm call of the reference's ConvNeXt block
 * (classification/fast/convnext.py:55) and the ln_row pattern (segmentation/fast/csrc/seg_kernels.cu:192-210). */
int fvm_layernorm_cl_f16(const void* x, const void* gamma, const void* beta, void* y, long long rows, int C, float eps,
                         long long ldx, long long ldy, void* stream);

/* fp32 or fp16 NCHW [N,C,H,W] (C <= 8) -> fp16 NHWC with channels zero-padded to 8 -- replaces clf::input_nhwc8
 * (fused_conv.cu:597-620, a template over float and __half inputs: one entry point per input type here). */
int fvm_input_nhwc8_f32(const float* x, void* y, int N, int C, int H, int W, void* stream);
int fvm_input_nhwc8_f16(const void* x, void* y, int N, int C, int H, int W, void* stream);

/* The same conversion into two column-parity planes per image row, y[n][h][w & 1][w >> 1][8] (W even): the input
 * layout of fvm_stem_conv_s2_f16. Same bytes as the NHWC8 tensor, columns regrouped. */
int fvm_input_nhwc8_split_f32(const float* x, void* y, int N, int C, int H, int W, void* stream);
int fvm_input_nhwc8_split_f16(const void* x, void* y, int N, int C, int H, int W, void* stream);

/* Stride-2 stem convolution on that layout: y[N,P,Q,K] (row stride ldy) = act(conv(x, w) + bias), w [K][R][S][8]
 * (input channels zero-padded to 8), padding (ph, pw) on both sides, stride 2 in both directions, R, S <= 8,
 * K % 8 == 0 and K <= 256. Replaces the reference's zero-padded 8-channel stem (classification/fast/fused.py:90-105,
 * run there through clf::conv_fused, fused_conv.cu:229-300): with the parity planes, consecutive output columns read
 * consecutive plane columns, so the input patch of a 16 x 8 block of outputs is staged once in shared memory and every
 * filter tap is a shifted view of it. */
int fvm_stem_conv_s2_f16(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int K, int R,
                         int S, int ph, int pw, long long ldy, int act, void* stream);

/* In place: y = relu?(y + bias[c] + res) -- replaces segx::bias_act_ (segmentation/fast/csrc/segx_ops.cu:28-42). */
int fvm_bias_act_f16(void* y, const void* bias, const void* res, long long pixels, int C, int relu, void* stream);

/* y = act(x * scale[c] + shift[c]), fp32 scale/shift -- replaces clf::affine_act (fused_conv.cu:308-335). */
int fvm_affine_act_f16(const void* x, const float* scale, const float* shift, void* y, long long pixels, int C,
                       long long ldx, long long ldy, int act, void* stream);

/* y = act(a + b) elementwise fp16 (fp32 math) -- the un-fused residual add the reference leaves to aten in MBConv
 * blocks (no custom kernel there: its rewritten EfficientNet-B4 graph keeps 25 aten adds). */
int fvm_add_act_f16(const void* a, const void* b, void* y, long long n, int act, void* stream);

/* PyTorch-exact bilinear resize of NHWC fp16 [N,h,w,C] -> [N,H,W,C] (align_corners both ways; sf_* <= 0 means derive
 * the scale from the sizes). If base != NULL: y = relu?(half(interp) + base) -- replaces segx::upsample_bilinear /
 * upsample_add (segmentation/fast/csrc/segx_ops.cu:59-157). */
int fvm_bilinear_f16(const void* x, const void* base, void* y, int N, int h, int w, int C, int H, int W, int align,
                     float sf_h, float sf_w, int relu, long long ldx, long long ldy, void* stream);

/* Fused bilinear upsample + channel argmax of NHWC fp16 scores [N,h,w,ld] (first C channels) -> int32 [N,H,W]; the
 * first maximum wins -- replaces segx::up_argmax (segx_ops.cu:171-195; seg_kernels.cu:11-42). */
int fvm_up_argmax_f16(const void* s, int32_t* out, int N, int h, int w, int C, long long ld, int H, int W, int align,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FVM_B200_H */
