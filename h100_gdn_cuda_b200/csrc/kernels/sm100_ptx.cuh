// Thin inline-PTX wrappers for the sm_100a features the Gated DeltaNet kernels use:
// mbarriers with bounded waits, TMA (cp.async.bulk[.tensor]) loads, tensor memory
// (tcgen05.alloc/ld/st), tcgen05.mma with shared-memory / tensor-memory operands, and
// the shared-memory and instruction descriptors those MMAs take.
//
// Every wait in this file is bounded: when the limit runs out the wait returns false
// and the caller records an error status instead of spinning forever.
#pragma once
#ifdef __CUDACC_RTC__
// NVRTC has no C library headers: spell the fixed-width types out.
typedef unsigned char uint8_t;
typedef unsigned short uint16_t;
typedef unsigned int uint32_t;
typedef int int32_t;
typedef unsigned long long uint64_t;
typedef long long int64_t;
typedef unsigned long long uintptr_t;
#else
#include <cuda_runtime.h>
#include <stdint.h>
#endif
#include <cuda_bf16.h>

namespace gdn {
namespace ptx {

#define GDN_DEVICE __device__ __forceinline__

GDN_DEVICE uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

GDN_DEVICE uint32_t elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}\n"
        : "=r"(pred));
    return pred;
}

// ------------------------------------------------------------------ mbarrier
GDN_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
GDN_DEVICE void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
GDN_DEVICE void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
GDN_DEVICE void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
GDN_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for the phase with the given parity to complete.  Gives up after about
// `kWaitLimitCycles` SM clock cycles (a couple of seconds), or at once when another thread of
// the CTA has already given up (`*abort_flag != 0`).  Returns false on give-up and sets the
// flag.  The clock is read only once in a while, so a wait that succeeds soon costs a handful
// of instructions.
constexpr long long kWaitLimitCycles = 4000ll * 1000ll * 1000ll;

GDN_DEVICE bool mbar_wait_limit(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit_cycles) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag != 0) return false;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}
GDN_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait_limit(bar, parity, abort_flag, kWaitLimitCycles);
}

// The same wait for warps that are not on a critical path: sleeps `kSleepNs` between polls so
// that the polling does not take issue slots and shared-memory queue entries from the warps
// that are.
template <unsigned kSleepNs>
GDN_DEVICE bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        __nanosleep(kSleepNs);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// ------------------------------------------------------------------ proxies / fences
GDN_DEVICE void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
GDN_DEVICE void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
GDN_DEVICE void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------ TMA loads
GDN_DEVICE void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
GDN_DEVICE void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1)
        : "memory");
}
GDN_DEVICE void tma_load_3d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "r"(c2)
        : "memory");
}
GDN_DEVICE void tma_load_4d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2,
                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// Warp-collective TMA loads: the converged warp calls them with warp-uniform arguments and one
// elected lane issues (keeps the tensor-map address and coordinates in uniform registers).
GDN_DEVICE void tma_load_4d_w(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
        "@pe cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];\n\t}\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
GDN_DEVICE void tma_load_2d_w(void* dst, const void* tmap, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
        "@pe cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];\n\t}\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
GDN_DEVICE void mbar_arrive_expect_tx_w(uint64_t* bar, uint32_t bytes) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
        "@pe mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}\n" ::"r"(smem_u32(bar)),
        "r"(bytes)
        : "memory");
}
// Pull a tile into L2 ahead of the load that will fetch it into shared memory.
GDN_DEVICE void tma_prefetch_4d(const void* tmap, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
GDN_DEVICE void tma_prefetch_2d(const void* tmap, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(c0), "r"(c1)
                 : "memory");
}
// Untiled counterpart: pull `bytes` (a multiple of 16) at a 16-byte aligned address into L2.
GDN_DEVICE void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(src)), "r"(bytes) : "memory");
}
// Programmatic dependent launch.  A kernel launched with programmatic stream serialization may
// start while the kernel before it in the stream is still running; `grid_dep_wait` blocks until that
// kernel has completed and its writes are visible (a no-op for an ordinary launch), and
// `grid_dep_launch` in the earlier kernel lets the later one be scheduled as SMs free up.
GDN_DEVICE void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
GDN_DEVICE void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
GDN_DEVICE void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// The same as a warp-collective call (warp-uniform arguments, one elected lane issues).
GDN_DEVICE void bulk_load_w(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
        "@pe cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t}\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ------------------------------------------------------------------ L2 cache policies for bulk copies
// evict_last: keep the lines in L2 as long as possible (data another kernel reads back soon);
// evict_first: drop them first (data streamed through once).
GDN_DEVICE uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
GDN_DEVICE uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
GDN_DEVICE void bulk_store_hint(void* dst, const void* src, uint32_t bytes, uint64_t policy) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(
                     reinterpret_cast<uint64_t>(dst)),
                 "r"(smem_u32(src)), "r"(bytes), "l"(policy)
                 : "memory");
}
// warp-collective (one elected lane issues), with an L2 policy
GDN_DEVICE void bulk_load_hint_w(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
        "@pe cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n\t}\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
GDN_DEVICE void tma_load_4d_hint_w(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2, int c3, uint64_t policy) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
        "@pe cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;\n\t}\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "l"(policy)
        : "memory");
}

// ------------------------------------------------------------------ TMA stores (shared -> global)
// Untiled bulk copy shared -> global (bulk-group completion); same alignment rules as bulk_load.
GDN_DEVICE void bulk_store(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                     reinterpret_cast<uint64_t>(dst)),
                 "r"(smem_u32(src)), "r"(bytes)
                 : "memory");
}
GDN_DEVICE void tma_store_4d(const void* tmap, const void* src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
GDN_DEVICE void tma_store_2d(const void* tmap, const void* src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1)
                 : "memory");
}
GDN_DEVICE void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's bulk groups still have to read their shared-memory source
template <int N>
GDN_DEVICE void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
GDN_DEVICE void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------ tensor memory
// One full warp allocates `ncols` (power of two >= 32) columns; the base address is
// written to `*slot` in shared memory.
GDN_DEVICE void tmem_alloc(uint32_t* slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(slot)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
GDN_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
GDN_DEVICE void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
GDN_DEVICE void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x (N x 32-bit) loads: thread i of the warp receives lane (base_lane + i),
// N consecutive columns.  The warp may only touch lanes 32*(warp_id % 4) .. +31.
GDN_DEVICE void tmem_ld8(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
GDN_DEVICE void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
GDN_DEVICE void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
GDN_DEVICE void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7])
        : "memory");
}
GDN_DEVICE void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
        : "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor for 128-byte-swizzled bf16 tiles.
//   K-major tile  : rows (M or N index) at a 128 B pitch, 64 bf16 of K per row;
//                   8-row groups `sbo` bytes apart (1024 when rows are packed).
//   MN-major tile : rows are K indices at a 128 B pitch holding 64 contiguous MN
//                   elements; 8-row groups `sbo` bytes apart; the next 64 MN elements
//                   start `lbo` bytes further on.
// Bits: [0,14) address>>4, [16,30) lbo>>4, [32,46) sbo>>4, [46,48) version=1,
//       [61,64) layout type (2 = 128-byte swizzle).
GDN_DEVICE uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
// Bits: [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format,
//       13 negate A, 14 negate B, 15 A is MN-major, 16 B is MN-major,
//       [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, bool a_mn_major,
                                                       bool b_mn_major, bool neg_a = false) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (neg_a ? (1u << 13) : 0u) |
           (a_mn_major ? (1u << 15) : 0u) | (b_mn_major ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ------------------------------------------------------------------ MMA (issued by ONE thread)
// D[tmem] (+)= A[smem] * B[smem]
GDN_DEVICE void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
GDN_DEVICE void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Variants with the accumulate flag fixed at compile time (no predicate set-up per MMA).
template <bool kAccumulate>
GDN_DEVICE void mma_ss_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    if (kAccumulate)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc)
                     : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc)
                     : "memory");
}
template <bool kAccumulate>
GDN_DEVICE void mma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    if (kAccumulate)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
                     "r"(a_tmem), "l"(b_desc), "r"(idesc)
                     : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
                     "r"(a_tmem), "l"(b_desc), "r"(idesc)
                     : "memory");
}
// Warp-collective variants: the whole (converged) warp calls them with warp-uniform operands
// and one elected lane issues the instruction.  Keeping the surrounding control flow
// warp-uniform lets the descriptors live in uniform registers, which is what the instruction
// consumes; issuing from inside an `if (lane == 0)` region costs tens of cycles per MMA in
// register moves.
template <bool kAccumulate>
GDN_DEVICE void mma_ss_w(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\t.reg .pred pa;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pa, %4, 0;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pa;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
template <bool kAccumulate>
GDN_DEVICE void mma_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\t.reg .pred pa;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pa, %4, 0;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pa;\n\t}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
// Eight K-steps (K = 128) of one accumulation as a single warp-collective issue: A from tensor
// memory (8 columns per step), B a K-major tile of two 64-column atoms 8192 bytes apart.  One
// election serves all eight instructions.
template <bool kAccumulateFirst>
GDN_DEVICE void mma_ts_k128_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\t.reg .pred pa;\n\t.reg .pred pt;\n\t.reg .b32 ta;\n\t.reg .b64 bd;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pa, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pa;\n\t"
        "add.u32 ta, %1, 8;\n\tadd.u64 bd, %2, 2;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 16;\n\tadd.u64 bd, %2, 4;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 24;\n\tadd.u64 bd, %2, 6;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 32;\n\tadd.u64 bd, %2, 512;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 40;\n\tadd.u64 bd, %2, 514;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 48;\n\tadd.u64 bd, %2, 516;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 56;\n\tadd.u64 bd, %2, 518;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "n"(kAccumulateFirst ? 1 : 0)
        : "memory");
}
// Four K-steps (K = 64) the same way; the B descriptor advances by `kStep16` 16-byte units per step
// (2 for a K-major tile, 128 for an MN-major one).
template <bool kAccumulateFirst, int kStep16>
GDN_DEVICE void mma_ts_k64_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\t.reg .pred pa;\n\t.reg .pred pt;\n\t.reg .b32 ta;\n\t.reg .b64 bd;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pa, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pa;\n\t"
        "add.u32 ta, %1, 8;\n\tadd.u64 bd, %2, %5;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 16;\n\tadd.u64 bd, %2, %6;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t"
        "add.u32 ta, %1, 24;\n\tadd.u64 bd, %2, %7;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], bd, %3, pt;\n\t}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "n"(kAccumulateFirst ? 1 : 0), "n"(kStep16), "n"(2 * kStep16),
        "n"(3 * kStep16)
        : "memory");
}
GDN_DEVICE void mma_commit_w(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(
            smem_u32(bar))
        : "memory");
}

// Descriptor of the same tile `bytes` further on (the start-address field counts 16-byte units;
// callers stay within the 256 KB the 14-bit field covers, so the add never carries out of it).
GDN_DEVICE uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }
// byte offset of K-step `ks` (16 bf16) inside a K-major tile of 64-column atoms `atom_bytes` apart
__host__ __device__ constexpr uint32_t kmajor_step(int ks, uint32_t atom_bytes) {
    return static_cast<uint32_t>(ks / 4) * atom_bytes + static_cast<uint32_t>(ks % 4) * 32u;
}

// Make `bar` complete one arrival when every MMA issued so far by this thread is done.
GDN_DEVICE void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// ------------------------------------------------------------------ small helpers
GDN_DEVICE uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low 16 bits), .y = hi
    return *reinterpret_cast<uint32_t*>(&v);
}
GDN_DEVICE float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
GDN_DEVICE float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Byte offset of element (row, col) of a bf16 tile stored as 128-byte rows of 64
// elements with the 128-byte swizzle TMA and tcgen05 use (16-byte chunk index XOR
// row % 8).  The tile base must be 1024-byte aligned.
GDN_DEVICE uint32_t sw128_offset(uint32_t row, uint32_t col) {
    const uint32_t chunk = (col >> 3) ^ (row & 7u);
    return row * 128u + chunk * 16u + (col & 7u) * 2u;
}

}  // namespace ptx
}  // namespace gdn
