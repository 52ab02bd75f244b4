// Thin wrappers over the sm_100a PTX this library uses: mbarrier, TMA (cp.async.bulk.tensor, never multicast),
// tcgen05 (TMEM allocation, MMA, commit, ld/st) and the shared-memory / instruction descriptors of tcgen05.mma.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mintb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// Programmatic dependent launch: a kernel launched with the "programmatic stream serialization" attribute may start while
// the kernel before it in the stream is still running; griddep_wait() returns once that kernel has completed and its writes
// are visible (at once when the attribute was not set).  griddep_launch() in the earlier kernel says that the later one may
// be scheduled as soon as every CTA of this grid has said so or has finished.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Non-blocking test of a phase, and a potentially blocking one (the hardware may suspend the thread for a short,
// implementation-defined time while the phase is pending).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The hint lets the hardware keep the thread suspended (no issue slots burnt on polling) until the phase completes or
// the time runs out; completion wakes it at once.
#ifndef MINTB_SUSPEND_NS
#define MINTB_SUSPEND_NS 20000
#endif
constexpr uint32_t kSuspendHintNs = MINTB_SUSPEND_NS;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: gives up once `limit_ns` (kWaitLimitNs for every wait of the library's kernels) of wall time have passed (checked every 1024 polls), records `code` in
// *status (if non-null) and returns false.  Callers unwind (skip the rest of their work, still release TMEM)
// instead of spinning forever.  The common case - the phase has already completed - costs one test.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, int* status, int code, uint64_t limit_ns) {
  if (mbar_test_wait(bar, parity)) return true;
#pragma unroll 1
  for (int it = 0; it < 1024; ++it)   // ordinary waits end here; the timer (slow to read) is not touched
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int it = 0; it < 1024; ++it)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) break;
  }
  if (status != nullptr) atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  return mbar_wait_limit(bar, parity, status, code, kWaitLimitNs);
}

// One thread per CTA calls this after its CTA's last draw from the work counter `ctr` = {next unit, CTAs that have left}:
// the last CTA of the grid clears the pair for the launch that gets it next.
__device__ __forceinline__ void leave_tile_counter(int* ctr, int n_ctas) {
  __threadfence();
  if (atomicAdd(ctr + 1, 1) == n_ctas - 1) {
    ctr[0] = 0;
    ctr[1] = 0;
    __threadfence();
  }
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load into this CTA's shared memory, completion counted in bytes on `bar`.  c0 (innermost) times the
// element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// 2-D tiled load (c0 innermost).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// 3-D tiled reduction shared memory -> global: every element of the box is ADDED to the tensor (type taken from the
// tensor map); rows outside the tensor are dropped.  Completion is tracked per thread in bulk groups.  c0 times the
// element size must be a multiple of 16 bytes and no coordinate may be negative.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// 2-D tiled store shared memory -> global (rows / columns outside the tensor are dropped); bulk-group completion.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all bulk groups of this thread have finished READING their shared-memory source (it may be overwritten)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all bulk groups of this thread except the most recent one have finished reading their shared-memory source
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// all bulk groups of this thread have completed
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Untiled bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.  Both addresses 16-byte
// aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate; one thread issues.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
// e4m3 x e4m3 -> fp32 (kind::f8f6f4, K = 32 per instruction)
__device__ __forceinline__ void umma_ss_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed (implies fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// TMEM address: lane in bits [16,32), column in bits [0,16).
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) { return base + (lane << 16) + col; }

#define MINTB_R8(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])
#define MINTB_W8(r, o) "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]), "r"(r[o + 6]), "r"(r[o + 7])

// 32 lanes x 32 bit, N consecutive columns: thread t of the warp receives lane (32 * (warp % 4) + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
      "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : MINTB_R8(r, 0), MINTB_R8(r, 8), MINTB_R8(r, 16), MINTB_R8(r, 24)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : MINTB_R8(r, 0), MINTB_R8(r, 8)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, "
      "%25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), MINTB_W8(r, 0), MINTB_W8(r, 8), MINTB_W8(r, 16), MINTB_W8(r, 24)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), MINTB_W8(r, 0), MINTB_W8(r, 8)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : MINTB_R8(r, 0)
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), MINTB_W8(r, 0)
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[N]) {
  static_assert(N == 4 || N == 8 || N == 16 || N == 32, "4, 8, 16 or 32 columns");
  if constexpr (N == 32) tmem_ld32(taddr, r);
  else if constexpr (N == 16) tmem_ld16(taddr, r);
  else if constexpr (N == 8) tmem_ld8(taddr, r);
  else tmem_ld4(taddr, r);
}
template <int N>
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[N]) {
  static_assert(N == 8 || N == 16 || N == 32, "8, 16 or 32 columns");
  if constexpr (N == 32) tmem_st32(taddr, r);
  else if constexpr (N == 16) tmem_st16(taddr, r);
  else tmem_st8(taddr, r);
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- descriptors
// Swizzle of a tile whose rows are `row_bytes` (32, 64 or 128) long and whose swizzle span equals the row.
enum Swizzle : uint32_t { kSw32 = 6, kSw64 = 4, kSw128 = 2 };
__host__ __device__ constexpr uint32_t swizzle_for_row_bytes(int row_bytes) {
  return row_bytes == 128 ? kSw128 : row_bytes == 64 ? kSw64 : kSw32;
}

// Shared-memory matrix descriptor: start address, leading/stride byte offsets (16-byte units), version 1, layout type.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= uint64_t((saddr >> 4) & 0x3FFF);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(layout) << 61;
  return d;
}
// The same descriptor split into 32-bit words for issue loops: a constant high word (stride offset, version, layout)
// and a low word = address field + leading-offset field, which advances by (bytes >> 4).
__host__ __device__ constexpr uint32_t desc_hi32(uint32_t sbo_bytes, uint32_t layout) {
  return ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (layout << 29);
}
__host__ __device__ constexpr uint32_t desc_lbo32(uint32_t lbo_bytes) { return ((lbo_bytes >> 4) & 0x3FFF) << 16; }
__device__ __forceinline__ uint32_t desc_addr32(uint32_t saddr) { return (saddr >> 4) & 0x3FFF; }
__device__ __forceinline__ uint64_t make_desc(uint32_t hi, uint32_t lo) { return (uint64_t(hi) << 32) | lo; }

// Operand whose reduction (K) dimension is contiguous: rows of `row_bytes` stacked at `row_bytes`, eight rows per
// swizzle atom.  One MMA consumes 32 bytes of each row; advance the start address by 32 bytes per K step.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr, int row_bytes) {
  return smem_desc(saddr, 16, 8 * row_bytes, swizzle_for_row_bytes(row_bytes));
}
// Operand whose M/N dimension is contiguous: each K index is one row of `row_bytes` (= the whole M/N extent if it fits
// one swizzle span, else `mn_block_stride` bytes separate consecutive spans).  One MMA consumes 16 rows.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr, int row_bytes, uint32_t mn_block_stride) {
  return smem_desc(saddr, mn_block_stride, 8 * row_bytes, swizzle_for_row_bytes(row_bytes));
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulate.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
         (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// Instruction descriptor for kind::f8f6f4 with e4m3 A/B (format code 0), both K-major, fp32 accumulate.
__host__ __device__ constexpr uint32_t idesc_e4m3(int M, int N) {
  return (1u << 4) | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a swizzled tile with rows of `row_bytes`
// (what TMA writes and tcgen05.mma reads): the chunk index is XOR-ed with the row's position in the 128-byte pattern.
__host__ __device__ constexpr uint32_t swizzled_offset(int row, int chunk, int row_bytes) {
  const uint32_t lin = uint32_t(row) * row_bytes + uint32_t(chunk) * 16;
  const uint32_t mask = row_bytes == 128 ? 7u : row_bytes == 64 ? 3u : 1u;
  return lin ^ (((lin >> 7) & mask) << 4);
}

}  // namespace ptx
}  // namespace mintb
