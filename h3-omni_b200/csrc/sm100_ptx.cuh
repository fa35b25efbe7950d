// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention
// kernels use: mbarriers with bounded waits, TMA tile loads, tensor memory
// (TMEM) allocation and access, and tcgen05 MMA issue/commit.
//
// Every wait in this file is bounded: after WAIT_LIMIT_NS without progress the
// waiter raises the CTA's abort word, the kernel records a status code in
// global memory and leaves through its normal teardown, so a protocol error
// shows up as an error status on the host and never as a hung GPU.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace h3b {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s per wait

// Status codes written to the device status word (first failure wins).
enum DeviceStatus : int {
    STATUS_OK = 0,
    STATUS_WAIT_TIMEOUT = 1,   // an mbarrier wait gave up
    STATUS_BAD_ARGUMENT = 2,   // a device-side bounds check refused an access
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// The same probe with a suspend-time hint: a probe that finds the phase incomplete parks the
// thread in hardware for up to `ns` nanoseconds (or until the phase completes) instead of coming
// straight back, so a long wait costs a few probes, not thousands of loop iterations.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return done != 0;
}
// Bounded wait for waits that are expected to be long (a softmax thread waiting for its next
// score tile, the producer waiting for a free slot): parked probes.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile int *abort_word) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long start = global_timer_ns();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait_parked(bar, parity, 4000u)) return true;
        if ((spin & 15u) == 0u) {
            if (*abort_word) return false;
            if (global_timer_ns() - start > WAIT_LIMIT_NS) {
                *abort_word = 1;
                return false;
            }
        }
    }
}

// Bounded wait. Returns false when the CTA is aborting (this waiter or another
// one ran out of time); `abort_word` lives in shared memory.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_word) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long start = global_timer_ns();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 0u) {
            if (*abort_word) return false;
            if (global_timer_ns() - start > WAIT_LIMIT_NS) {
                *abort_word = 1;
                return false;
            }
        }
    }
}

// Warp-collective bounded wait: lane 0 polls, the warp gets the result. 32x fewer probes of
// the mbarrier word than every lane polling for itself - the probes go to shared memory,
// which the tensor core is reading its operands from at the same time.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_word) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_word);
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}

// The same with the loop run by the whole warp and only the probe predicated on lane 0: no
// divergent loop, so the registers of a register-heavy caller stay where they are.
__device__ __forceinline__ bool mbar_wait_uniform(uint32_t bar, uint32_t parity, volatile int *abort_word) {
    const bool prober = (threadIdx.x & 31) == 0;
    unsigned long long start = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done = 0;
        if (prober) done = mbar_try_wait(bar, parity) ? 1u : 0u;
        if (__shfl_sync(0xffffffffu, done, 0)) return true;
        if ((spin & 255u) == 255u) {
            uint32_t stop = 0;
            if (prober) {
                const unsigned long long now = global_timer_ns();
                if (!start) start = now;
                if (*abort_word) stop = 1;
                else if (now - start > WAIT_LIMIT_NS) {
                    *abort_word = 1;
                    stop = 1;
                }
            }
            if (__shfl_sync(0xffffffffu, stop, 0)) return false;
        }
    }
}

// Lane 0 polls, the other lanes wait for it at a warp barrier; the outcome travels through the
// abort word (a wait only fails by raising it), so no shuffle is needed.
__device__ __forceinline__ bool mbar_wait_lane0(uint32_t bar, uint32_t parity, volatile int *abort_word) {
    if ((threadIdx.x & 31) == 0) mbar_wait(bar, parity, abort_word);
    __syncwarp();
    return *abort_word == 0;
}

// For a converged warp whose lanes all wait for the same barrier: when the barrier is already
// complete this is one probe per lane (one broadcast access for the warp) and nothing else;
// otherwise every lane polls and the warp agrees on the outcome.
__device__ __forceinline__ bool mbar_wait_converged(uint32_t bar, uint32_t parity, volatile int *abort_word) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_word));
}

// One lane of a converged warp (the predicate form the compiler recognises as "uniform code,
// one lane acts": address arithmetic around it stays in the uniform datapath).
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(chosen));
    return chosen != 0;
}

// ---- TMA (non-multicast tile loads only) ---------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *map, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// ---- tensor memory -------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tc5_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc5_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane
// (warp%4)*32 + t, registers r[0..31] = columns col..col+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---- tcgen05 MMA -----------------------------------------------------------------
// Shared-memory matrix descriptor for a 128-byte-swizzled bf16/fp16 tile whose
// rows are 128 bytes (64 elements) and whose 8-row groups are 1024 bytes apart.
//   K-major operand  : lbo is ignored by the hardware (set to 16 B), sbo = 1024.
//   MN-major operand : lbo = byte distance between consecutive 64-element
//                      chunks along MN, sbo = 1024 (next 8 rows along K).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version for sm_100
    d |= (uint64_t)2 << 61;  // 128-byte swizzle
    return d;
}
// Instruction descriptor, kind::f16, fp32 accumulate, A K-major.
//   ab_format: 0 = fp16, 1 = bf16. b_mn_major: B operand is MN-major.
__host__ __device__ constexpr uint32_t mma_idesc(uint32_t m, uint32_t n, uint32_t ab_format,
                                                 uint32_t b_mn_major) {
    return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (b_mn_major << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same two instructions with the 64-bit shared-memory descriptors passed as (low, high)
// words. Consecutive K-steps of one tile differ only in the address field of the low word, so
// the issuing thread builds a descriptor once per tile and spends one 32-bit add per MMA - it
// shares its scheduler with busy softmax warps and every instruction it saves shortens the
// time the tensor pipe waits for work.
__device__ __forceinline__ void mma_ss_words(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                             uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ts_words(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                             uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// Register re-allocation between warpgroups (four aligned warps execute it together).
template <int REGS>
__device__ __forceinline__ void warpgroup_reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void warpgroup_reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace h3b
