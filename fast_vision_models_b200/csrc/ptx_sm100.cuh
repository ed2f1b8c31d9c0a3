// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc, MMA, commit, ld).
// Every wait is bounded: a wait that does not complete within WAIT_LIMIT_NS records a status word and returns false,
// so a broken barrier protocol ends the kernel with an error code instead of hanging the GPU.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace fvm {

static constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}
// Non-blocking test of a phase (mbarrier.test_wait): used to look ahead at the barrier of the next step while the
// current one is being issued, so that the round trip to shared memory is off the critical path.
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}
// Bounded wait. `abort_flag` is a word in shared memory shared by all roles of the CTA: the first role that gives up
// sets it (and the caller records a status code); the other roles see it on their next poll and leave too.
// BACKOFF_NS > 0 puts the warp to sleep between polls: many-lane waiters (epilogue warps) then leave the issue slots
// of their scheduler to the single-thread producer / MMA roles instead of spinning next to them.
template <int BACKOFF_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;      // another wait of this CTA already gave up: do not wait again
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    for (;;) {
        if (BACKOFF_NS > 0) __nanosleep(BACKOFF_NS);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 0xff) == 0) {
            if (*abort_flag) return false;
            unsigned long long now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) { *abort_flag = 1; return false; }
        }
    }
}

// Division by a run-time constant as multiply-high + shift (valid for numerators below 2^31); `mul`/`shr` from
// fastdiv_init on the host.
struct FastDiv {
    uint32_t div, mul, shr;
};
__host__ inline FastDiv fastdiv_init(uint32_t d) {
    FastDiv f;
    f.div = d;
    if (d <= 1) {
        f.mul = 0;
        f.shr = 0;
        return f;
    }
    uint32_t lg = 0;
    while ((1ull << lg) < d) ++lg;
    const uint32_t p = 31 + lg;
    f.mul = static_cast<uint32_t>(((1ull << p) + d - 1) / d);
    f.shr = p - 32;
    return f;
}
__device__ __forceinline__ uint32_t fastdiv(uint32_t n, const FastDiv& f) {
    return f.div <= 1 ? n : (__umulhi(n, f.mul) >> f.shr);
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const void* desc) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(desc)) : "memory");
}
// L2 eviction priorities for bulk loads (0 = none): evict_first for data that is dead after this read, so that it does
// not push out lines a later kernel will want; evict_last for the opposite.
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ unsigned long long l2_policy_evict_last() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1,
                                            unsigned long long policy = 0) {
    if (policy) {
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
            : "memory");
        return;
    }
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1, int c2, int c3,
                                            unsigned long long policy = 0) {
    if (policy) {
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
            : "memory");
        return;
    }
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
// im2col-mode load of NHWC activations: coordinates (c, w, h, n) of the first pixel's filter-window origin, plus the
// filter tap offset (off_w, off_h) in input pixels (tap index times dilation).
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const void* desc, uint32_t bar, int c, int w, int h,
                                                   int n, uint16_t off_w, uint16_t off_h, unsigned long long policy = 0) {
    if (policy) {
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8}, %9;"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
            "h"(off_h), "l"(policy)
            : "memory");
        return;
    }
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
        "h"(off_h)
        : "memory");
}

// Bulk tensor store shared -> global (clipped at the tensor bounds), tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void tma_store_2d(const void* desc, uint32_t src, int c0, int c1, unsigned long long policy = 0) {
    if (policy) {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
                     ::"l"(reinterpret_cast<uint64_t>(desc)), "r"(src), "r"(c0), "r"(c1), "l"(policy)
                     : "memory");
        return;
    }
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(desc)), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* desc, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(desc)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* desc, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(desc)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until every committed bulk store of this thread has finished READING shared memory (the source may be reused).
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Orders this thread's generic-proxy writes to shared memory before later async-proxy (TMA) reads of them.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Two fp32 values in one 64-bit register and packed arithmetic on them (sm_100 executes add.f32x2 as one instruction).
__device__ __forceinline__ unsigned long long f2_pack(uint32_t lo, uint32_t hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// (lo, hi) fp32 pair -> one fp16x2 word, round to nearest even
__device__ __forceinline__ uint32_t f2_to_h2(unsigned long long v) {
    float lo, hi;
    f2_unpack(v, lo, hi);
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// fp16x2 word -> (lo, hi) fp32 pair
__device__ __forceinline__ unsigned long long h2_to_f2(uint32_t h) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    return f2_pack(__float_as_uint(f.x), __float_as_uint(f.y));
}
__device__ __forceinline__ uint32_t h2_relu(uint32_t h) {
    uint32_t r;
    asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(h), "r"(0u));
    return r;
}
__device__ __forceinline__ unsigned long long f2_mul(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long f2_splat(float c) {
    return f2_pack(__float_as_uint(c), __float_as_uint(c));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// SiLU of an fp32 pair: x sigmoid(x) = x (0.5 + 0.5 tanh(x / 2)) = hx + hx tanh(hx) with hx = x / 2: two packed
// instructions and ONE special-function instruction per element (tanh.approx.f32, relative error about 2^-11, the size
// of an fp16 rounding step). Measured on B200 against x / (1 + 2^(-x log2 e)) (ex2 + rcp per element): 1x1 24 -> 144 at
// 190x190, batch 64: 231 -> 197 us, EfficientNet-B4 forward 5.45 -> 5.16 ms; the epilogue warps are bound by
// instruction issue, so what counts is the instruction count (a reciprocal by Newton steps on the FMA pipe was slower:
// 306 us; a packed-fp16 tanh was faster still but doubled the network's error against the oracle).
__device__ __forceinline__ float tanh_approx(float x) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ unsigned long long f2_silu(unsigned long long x) {
    float lo, hi;
    const unsigned long long hx = f2_mul(x, f2_splat(0.5f));
    f2_unpack(hx, lo, hi);
    const unsigned long long t = f2_pack(__float_as_uint(tanh_approx(lo)), __float_as_uint(tanh_approx(hi)));
    return f2_fma(hx, t, hx);
}
// (a0, a1) += the two halves of an fp16x2 word, in fp32: the mixed-precision add of sm_100 converts and adds in one
// instruction per element (no separate fp16 -> fp32 conversion).
__device__ __forceinline__ void f32_add_h2(float& a0, float& a1, uint32_t h2) {
    asm("{\n\t"
        ".reg .b16 lo, hi;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "add.rn.f32.f16 %0, lo, %0;\n\t"
        "add.rn.f32.f16 %1, hi, %1;\n\t"
        "}\n"
        : "+f"(a0), "+f"(a1)
        : "r"(h2));
}
// GELU (erf form) of an fp32 pair: gelu(x) = max(x, 0) - |x| erfc(|x| / sqrt 2) / 2  (for x >= 0 this is
// x (2 - erfc) / 2, for x < 0 it is x erfc / 2). log2(erfc(a / sqrt 2)) is smooth, so erfc comes from ONE special-function
// instruction per element: 2^Q(a) with Q a degree-6 polynomial without constant term, least-squares fitted on Chebyshev
// nodes of a = |x| in [0, 5.94] (relative error of erfc below 5e-5; |x| erfc / 2 within 7.1e-6 of the exact value,
// checked over 200 001 points up to |x| = 12, where a is clamped to 5.94 and the term is below 2e-8 anyway). The
// polynomial runs on packed pairs. The previous form (Abramowitz & Stegun 7.1.26) needed a reciprocal and an exponential
// per element, and the special-function unit (16 results per clock per SM) was what bounded a GELU epilogue.
__device__ __forceinline__ unsigned long long f2_gelu_erf(unsigned long long x) {
    float xl, xh;
    f2_unpack(x, xl, xh);
    const float al = fminf(fabsf(xl), 5.9397f), ah = fminf(fabsf(xh), 5.9397f);
    const unsigned long long a = f2_pack(__float_as_uint(al), __float_as_uint(ah));
    unsigned long long q = f2_fma(f2_splat(2.377673263e-05f), a, f2_splat(-6.253862521e-04f));
    q = f2_fma(q, a, f2_splat(7.295017131e-03f));
    q = f2_fma(q, a, f2_splat(-5.151612312e-02f));
    q = f2_fma(q, a, f2_splat(-4.607414007e-01f));
    q = f2_fma(q, a, f2_splat(-1.150532007e+00f));
    q = f2_fma(q, a, f2_splat(-1.0f));               // Q(a) - 1: the exponent of erfc / 2
    float ql, qh;
    f2_unpack(q, ql, qh);
    // |x| erfc / 2 >= 0, with the unclamped |x|
    const float hl = fabsf(xl) * ex2_approx(ql), hh = fabsf(xh) * ex2_approx(qh);
    return f2_pack(__float_as_uint(fmaxf(xl, 0.f) - hl), __float_as_uint(fmaxf(xh, 0.f) - hh));
}
// 16 bytes of shared memory as two fp32 pairs. Not volatile: only for data that is constant while the kernel's
// roles run (the bias copy), so the compiler may schedule it freely.
__device__ __forceinline__ void lds_2xf2(uint32_t addr, unsigned long long& a, unsigned long long& b) {
    asm("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(addr));
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; one thread issues. `accumulate` = 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One lane of a converged warp, the same one on every call (elect.sync over the full mask). The compiler knows that a
// region guarded by this predicate runs in a single lane and keeps the operands of the single-thread tcgen05 / TMA
// instructions in uniform registers: measured on B200, a loop of tcgen05.mma issued under `if (elect_one())` costs
// about 50 cycles per instruction, the same loop under `if (lane == 0)` about 120.
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, e;\n\t"
        "}\n"
        : "=r"(pred));
    return pred;
}
// One tcgen05.mma with descriptors given as (low word, high word). Call from the single issuing lane.
__device__ __forceinline__ void umma_f16_words(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Four tcgen05.mma whose A and B descriptors advance by constant steps (low words): the four tap pairs of one filter
// column in stem mode. The first accumulates iff `acc0` != 0. Call from the single issuing lane.
__device__ __forceinline__ void umma_f16_stepped4(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t a_step, uint32_t b_lo,
                                                  uint32_t b_hi, uint32_t b_step, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 al, bl;\n\t"
        "setp.ne.b32 p, %8, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%4, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
        "add.u32 al, %1, %3;\n\t"
        "add.u32 bl, %4, %6;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, 1;\n\t"
        "add.u32 al, al, %3;\n\t"
        "add.u32 bl, bl, %6;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, 1;\n\t"
        "add.u32 al, al, %3;\n\t"
        "add.u32 bl, bl, %6;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, 1;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(a_step), "r"(b_lo), "r"(b_hi), "r"(b_step), "r"(idesc), "r"(acc0)
        : "memory");
}
// The four tcgen05.mma of one 64-half k-block (K = 16 each) as one instruction sequence. Descriptors come as (low word,
// high word): the start address lives in the low word, so the steps along K (+32 bytes = +2) are 32-bit adds. The first
// MMA accumulates iff `acc0` != 0, the other three always do. Call from the single issuing lane.
__device__ __forceinline__ void umma_f16_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 al, bl;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
        "add.u32 al, %1, 2;\n\t"
        "add.u32 bl, %3, 2;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, 1;\n\t"
        "add.u32 al, %1, 4;\n\t"
        "add.u32 bl, %3, 4;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, 1;\n\t"
        "add.u32 al, %1, 6;\n\t"
        "add.u32 bl, %3, 6;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, 1;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(acc0)
        : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has finished (implies fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets TMEM lane (lane_base + i), r[j] = column base + j.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
        "[%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes (64 halves) wide, written by TMA
// with the 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO); LBO is unused for swizzled K-major layouts.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);        // start address, bits [0,14)
    d |= static_cast<uint64_t>(1) << 16;                           // leading byte offset (ignored), bits [16,30)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset, bits [32,46)
    d |= static_cast<uint64_t>(1) << 46;                           // descriptor version 1 (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                           // layout type: SWIZZLE_128B
    return d;
}
// As umma_desc_sw128 for an operand that starts at any 128-byte row of a swizzled block (not only at a 1024-byte
// boundary) and whose 8-row groups are `sbo` bytes apart. The hardware applies the swizzle to the absolute
// shared-memory address, so data written by TMA into a 1024-byte-aligned buffer is read back correctly from any row
// with the base-offset field left at zero (measured on B200: a non-zero base offset gives wrong operands here).
__device__ __forceinline__ uint64_t umma_desc_sw128_at(uint32_t smem_addr, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3fff) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// K-major operand tile whose rows are 32 bytes (16 halves = one MMA K step) wide, written by TMA with the 32-byte
// swizzle: 8-row groups are 256 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw32(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(256 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(6) << 61;                           // layout type: SWIZZLE_32B
    return d;
}
// K-major tile without swizzle ("interleaved"): core matrices of 8 rows x 16 bytes stored contiguously (128 bytes);
// `sbo` = byte distance between 8-row groups, `lbo` = byte distance between the two 16-byte K halves of one MMA.
__device__ __forceinline__ uint64_t umma_desc_interleaved(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3fff) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}
// Instruction descriptor for kind::f16: fp16 A and B (both K-major), fp32 accumulator, M x N tile.
__host__ __device__ inline uint32_t umma_idesc_f16_f32(int m, int n) {
    uint32_t d = 0;
    d |= 1u << 4;                               // accumulator format: f32
    d |= 0u << 7;                               // A: f16
    d |= 0u << 10;                              // B: f16
    d |= static_cast<uint32_t>(n >> 3) << 17;   // N / 8
    d |= static_cast<uint32_t>(m >> 4) << 24;   // M / 16
    return d;
}

// ---------------------------------------------------------------- CTA pairs (thread-block clusters of two)
// A pair of CTAs on neighbouring SMs shares one MMA: tcgen05.mma.cta_group::2 with M = 256 is issued by one thread of
// the even CTA, reads rows 0..127 of A and the first N/2 rows of B from that CTA's shared memory and rows 128..255 /
// the second N/2 rows of B from the odd CTA's (same shared-memory offsets in both), and leaves rows 0..127 of D in the
// even CTA's TMEM and rows 128..255 in the odd CTA's. Each SM therefore fetches only half of the B tile.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// All threads of all CTAs of the cluster (also a CTA-wide barrier); release / acquire at cluster scope.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrivals on an mbarrier of another CTA of the cluster (`bar` from mapa_shared). Default semantics (release at CTA
// scope), as for the local forms: what crosses the pair is ordered by the tcgen05 fences and the async proxy, and a
// cluster-scope acquire in the MMA thread's waits cost about 0.7 us per k-block when it was tried.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// Bulk tensor loads whose completion is counted on an mbarrier of either CTA of the pair (`bar`: a shared::cluster
// address); the destination is this CTA's shared memory: each CTA fetches its own boxes.
__device__ __forceinline__ void tma_pair_load_2d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1,
                                                 unsigned long long policy = 0) {
    if (policy) {
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
            : "memory");
        return;
    }
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_pair_load_3d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_pair_load_im2col_4d(uint32_t dst, const void* desc, uint32_t bar, int c, int w, int h,
                                                        int n, uint16_t off_w, uint16_t off_h, unsigned long long policy = 0) {
    if (policy) {
        asm volatile(
            "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8}, %9;"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
            "h"(off_h), "l"(policy)
            : "memory");
        return;
    }
    asm volatile(
        "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
        "h"(off_h)
        : "memory");
}
// TMEM of both CTAs of the pair: executed by the same warp of each CTA with the same arguments.
__device__ __forceinline__ void tmem_pair_alloc(uint32_t smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_pair_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_pair_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// The four MMAs (256 x N x 16 each, over both CTAs) of one 64-half k-block; see umma_f16_kblock.
__device__ __forceinline__ void umma_pair_f16_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                     uint32_t b_hi, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 al, bl;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t"
        "add.u32 al, %1, 2;\n\t"
        "add.u32 bl, %3, 2;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, 1;\n\t"
        "add.u32 al, %1, 4;\n\t"
        "add.u32 bl, %3, 4;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, 1;\n\t"
        "add.u32 al, %1, 6;\n\t"
        "add.u32 bl, %3, 6;\n\t"
        "mov.b64 da, {al, %2};\n\t"
        "mov.b64 db, {bl, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, 1;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(acc0)
        : "memory");
}
// Arrive on an mbarrier of either CTA of the pair (`bar`: shared::cluster address) once every pair MMA issued so far
// by this thread has finished.
__device__ __forceinline__ void umma_pair_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------- activations shared by every kernel
// Codes follow the reference's act_f (classification/fast/csrc/fused_conv.cu:33-43):
// 0 none, 1 relu, 2 relu6, 3 silu, 4 hardswish, 5 gelu (erf), 6 gelu (tanh).
__device__ __forceinline__ float act_f(float v, int act) {
    switch (act) {
        case 1: return fmaxf(v, 0.f);
        case 2: return fminf(fmaxf(v, 0.f), 6.f);
        case 3: return v / (1.f + __expf(-v));
        case 4: return v * fminf(fmaxf(v + 3.f, 0.f), 6.f) * (1.f / 6.f);
        case 5: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        case 6: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    }
    return v;
}

}  // namespace fvm
