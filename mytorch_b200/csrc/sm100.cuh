// sm_100a building blocks in inline PTX: mbarrier, TMA tile loads (never
// multicast), tcgen05 tensor-memory allocation / MMA / commit / load, and the
// shared-memory and instruction descriptors tcgen05.mma consumes.
//
// Every wait is bounded: after ~2 s of SM clock a wait gives up, raises the
// CTA-wide abort flag and returns false; callers then leave their loops, join
// at the common teardown and free tensor memory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {
namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

constexpr long long kWaitLimitCycles = 4000000000ll;  // ~2 s at 2 GHz

// Waits for the phase with the given parity to complete. `abort_flag` is a
// shared-memory int that any role sets when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 255) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) { *abort_flag = 1; return false; }
    }
  }
  return true;
}

// ---- programmatic dependent launch -------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while
// the kernel before it in the stream still runs; griddep_wait() returns once that
// kernel has completed and its writes are visible, and must precede every access
// to global memory. griddep_launch() lets the NEXT kernel in the stream start its
// own prologue as soon as every CTA of this one has passed the call.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- TMA: 2-D tiled load global -> shared, completion on an mbarrier ---------
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// Brings the box into L2 without a destination in shared memory: a later tma_load_4d of the same
// box finds it there.
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* map, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global [%0, {%1, %2, %3, %4}];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
// 2-D tiled store / reduce-add shared -> global through a tensor map (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src_smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src_smem, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src_smem, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, uint32_t src_smem, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory ----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], fp16/bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with the A operand read from tensor memory (K-major, lane = row, 32-bit
// columns of packed half pairs) instead of shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four / eight MMAs into one accumulator from one asm statement, all operands ready in
// registers: after the barrier wait that precedes them the issuing thread executes nothing but
// the MMAs themselves. (That thread shares a scheduler with busy warps and advances only every
// 10-20 cycles, so every instruction between the wait and the last MMA delays the tensor pipe.)
// The first MMA overwrites the accumulator unless acc_first != 0; the others accumulate.
__device__ __forceinline__ void umma_f16_x4(uint32_t d, const uint64_t* a, const uint64_t* b, uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n"
      ".reg .pred p, pt;\n"
      "setp.ne.b32 p, %10, 0;\n"
      "setp.eq.b32 pt, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %9, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %4, %9, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %6, %9, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %8, %9, pt;\n"
      "}\n"
      ::"r"(d), "l"(a[0]), "l"(b[0]), "l"(a[1]), "l"(b[1]), "l"(a[2]), "l"(b[2]), "l"(a[3]), "l"(b[3]), "r"(idesc), "r"(acc_first)
      : "memory");
}
__device__ __forceinline__ void umma_f16_x8(uint32_t d, const uint64_t* a, const uint64_t* b, uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n"
      ".reg .pred p, pt;\n"
      "setp.ne.b32 p, %18, 0;\n"
      "setp.eq.b32 pt, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %17, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %4, %17, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %6, %17, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %8, %17, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %10, %17, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %11, %12, %17, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %13, %14, %17, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %15, %16, %17, pt;\n"
      "}\n"
      ::"r"(d), "l"(a[0]), "l"(b[0]), "l"(a[1]), "l"(b[1]), "l"(a[2]), "l"(b[2]), "l"(a[3]), "l"(b[3]),
        "l"(a[4]), "l"(b[4]), "l"(a[5]), "l"(b[5]), "l"(a[6]), "l"(b[6]), "l"(a[7]), "l"(b[7]), "r"(idesc), "r"(acc_first)
      : "memory");
}
// Eight MMAs with the A operand in tensor memory: columns a_tmem, a_tmem + 8, ... (16 half
// elements of K per step).
__device__ __forceinline__ void umma_f16_ts_x8(uint32_t d, uint32_t a_tmem, const uint64_t* b, uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n"
      ".reg .pred p, pt;\n"
      ".reg .b32 a1, a2, a3, a4, a5, a6, a7;\n"
      "setp.ne.b32 p, %11, 0;\n"
      "setp.eq.b32 pt, 0, 0;\n"
      "add.u32 a1, %1, 8;\n"
      "add.u32 a2, %1, 16;\n"
      "add.u32 a3, %1, 24;\n"
      "add.u32 a4, %1, 32;\n"
      "add.u32 a5, %1, 40;\n"
      "add.u32 a6, %1, 48;\n"
      "add.u32 a7, %1, 56;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %10, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], %3, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], %4, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], %5, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a4], %6, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a5], %7, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a6], %8, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a7], %9, %10, pt;\n"
      "}\n"
      ::"r"(d), "r"(a_tmem), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7]),
        "r"(idesc), "r"(acc_first)
      : "memory");
}
// The same with the A operand in four separate pieces of 16 columns (two steps each) that start 32
// columns apart: columns a_tmem, +8, +32, +40, +64, +72, +96, +104.
__device__ __forceinline__ void umma_f16_ts_x8_pairs(uint32_t d, uint32_t a_tmem, const uint64_t* b, uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n"
      ".reg .pred p, pt;\n"
      ".reg .b32 a1, a2, a3, a4, a5, a6, a7;\n"
      "setp.ne.b32 p, %11, 0;\n"
      "setp.eq.b32 pt, 0, 0;\n"
      "add.u32 a1, %1, 8;\n"
      "add.u32 a2, %1, 32;\n"
      "add.u32 a3, %1, 40;\n"
      "add.u32 a4, %1, 64;\n"
      "add.u32 a5, %1, 72;\n"
      "add.u32 a6, %1, 96;\n"
      "add.u32 a7, %1, 104;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %10, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], %3, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], %4, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], %5, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a4], %6, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a5], %7, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a6], %8, %10, pt;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a7], %9, %10, pt;\n"
      "}\n"
      ::"r"(d), "r"(a_tmem), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7]),
        "r"(idesc), "r"(acc_first)
      : "memory");
}
// Makes `bar` complete once all MMAs issued so far by this thread have finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Loads 32 consecutive fp32 columns of this warp's 32 TMEM lanes (lane = row).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Stores 32 consecutive fp32 columns of this warp's 32 TMEM lanes.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// Stores 16 consecutive 32-bit columns of this warp's 32 TMEM lanes.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- CTA pairs (cluster of two CTAs sharing one MMA, cta_group::2) ------------
// The even CTA of the pair (cluster rank 0) issues the MMAs; each CTA supplies
// its own 128 rows of A and half of the B tile from its own shared memory and
// receives its 128 rows of the accumulator in its own tensor memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {   // every thread of both CTAs
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tile load whose completion is counted on a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_smem, uint32_t ncols) {  // one warp in each CTA
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Completion of the pair's MMAs issued so far arrives on the barrier at this
// shared-memory offset in both CTAs (a barrier signal, not a data copy).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}

// ---- descriptors ------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, for a tile whose rows are
// 128 bytes (64 half elements) and whose base is 1024-byte aligned.
//   K-major operand  (rows = M/N index, 128 B of K per row): SBO = 1024 B
//     between groups of 8 rows; advance K by 16 elements = +32 B.
//   MN-major operand (rows = K index, 128 B = 64 M/N elements per row): LBO =
//     byte distance between 64-element M/N chunks, SBO = 1024 B between groups
//     of 8 K rows; advance K by 16 = +2048 B.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16: fp32 accumulator, A/B format
// (0 = f16, 1 = bf16), operand majors (0 = K-major, 1 = MN-major), shape MxN.
__host__ __device__ inline uint32_t idesc_f16(int ab_format, int a_mn_major, int b_mn_major, int M, int N) {
  uint32_t d = 0;
  d |= 1u << 4;                          // D format: f32
  d |= (uint32_t)ab_format << 7;         // A format
  d |= (uint32_t)ab_format << 10;        // B format
  d |= (uint32_t)(a_mn_major ? 1 : 0) << 15;
  d |= (uint32_t)(b_mn_major ? 1 : 0) << 16;
  d |= (uint32_t)(N >> 3) << 17;
  d |= (uint32_t)(M >> 4) << 24;
  return d;
}

}  // namespace sm100

// Host side: cuTensorMapEncodeTiled reached through the runtime (the library
// does not link libcuda). Describes a 2-D row-major half/bf16 matrix
// [outer, inner] with row stride `ld` elements; box = box_inner x box_outer,
// 128-byte swizzle, out-of-range elements read as zero.
int make_tmap_2d(CUtensorMap* map, const void* base, int is_bf16, uint64_t inner, uint64_t outer,
                 uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer);
// General form, up to 4 dims (dims[0] innermost; strides in elements for dims 1..rank-1).
int make_tmap_nd(CUtensorMap* map, const void* base, int is_bf16, int rank, const uint64_t* dims,
                 const uint64_t* strides_elems, const uint32_t* box);
// 2-D map over a row-major matrix of any library dtype (mt_dtype code), for TMA stores.
// N-d map of any library dtype (dims[0] innermost, strides in elements for dims 1..rank-1).
int make_tmap_nd_typed(CUtensorMap* map, const void* base, int mt_dtype_code, int rank, const uint64_t* dims,
                       const uint64_t* strides_elems, const uint32_t* box);
int make_tmap_2d_typed(CUtensorMap* map, const void* base, int mt_dtype_code, uint64_t inner, uint64_t outer,
                       uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer);

}  // namespace mt
