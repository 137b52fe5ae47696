// Blackwell (sm_100a) primitives used by the tcgen05 kernels: mbarrier with bounded waits,
// TMA tile loads (each CTA fetches its own tiles; no kernel here uses clusters), TMEM allocation, tcgen05.mma / ld / commit,
// shared-memory and instruction descriptors.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace bsrl {
namespace tc5 {

// The library keeps one device status word per GPU: 0 = fine, otherwise the code of the first
// bounded wait that ran out (kernel id * 16 + role).  Kernels get its address as an argument;
// bsrl_device_status() reads and clears it.

constexpr uint32_t kSpinLimit = 1u << 21;  // try_wait polls before a wait gives up (a fraction of a second)

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when `limit` polls ran out or another role already gave up (*abort != 0).
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;   // the hardware parks the thread inside try_wait
    if ((i & 1023u) == 1023u && *abort) return false;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort) {
  return mbar_wait_limit(bar, parity, abort, kSpinLimit);
}

// Whole-warp bounded wait: only lane 0 polls the barrier (32 lanes polling the same word would
// compete with the tensor core's operand reads for shared-memory bandwidth); the outcome is
// broadcast.  Must be called by all 32 lanes.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// 2-D TMA tile load global -> shared (this CTA only), completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// 2-D tile store shared -> global (bulk async group of the issuing thread); rows / columns past the
// tensor's extent are clipped
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
// 3-D forms (x = column, y = token of the env, z = env): rows past a dimension's extent are zero-filled
// by the load and clipped by the store
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int x, int y, int z, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of this thread's bulk groups still have to READ their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// waits until all of this thread's bulk groups are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D(tmem, 128 x N f32) (+)= A(smem) * B(smem)^T, fp16 operands, issued by one thread
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D(tmem) (+)= A(tmem) * B(smem)^T: the A operand (128 rows x 16 fp16, two per 32-bit column, 8 columns)
// comes from tensor memory, only B is fetched from shared memory
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread = lane = row)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile stored as [rows][64 fp16] with the
// 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are
// 1024 bytes apart; the tile base is 1024-byte aligned; a 16-element K step advances the start
// address by 32 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major): 1
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;            // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;            // layout: 128-byte swizzle
  return d;
}

// Descriptor of an MN-major operand tile: the contraction index runs over 128-byte ROWS of 64 fp16
// along M (or N), 128-byte swizzle, as a TMA load of a {64 columns, k rows, blocks} box writes it:
// 8-row groups (8 steps of the contraction index) are 1024 bytes apart, the next 64-column block of
// M / N starts block_bytes further on.  A 16-step K slice advances the start address by 2048 bytes.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t block_bytes) {
  uint64_t d = (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((block_bytes >> 4) & 0x3FFF) << 16;   // leading byte offset: between 64-column blocks
  d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: between 8-row groups
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: f16 x f16 -> f32, M = 128, N = n (n % 16 == 0); both operands K-major
// unless a_mn / b_mn say that operand is MN-major
__host__ __device__ inline uint32_t idesc_f16(int m, int n, int a_mn = 0, int b_mn = 0) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(a_mn ? 1 : 0) << 15) | ((uint32_t)(b_mn ? 1 : 0) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// byte offset of element (row, col) inside a [rows][64 fp16] 128-byte-swizzled tile
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  uint32_t chunk = (uint32_t)(col >> 3) ^ (uint32_t)(row & 7);
  return (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u + chunk * 16u + (uint32_t)(col & 7) * 2u;
}

}  // namespace tc5

// Encodes a 2-D fp16 row-major (rows, cols) tensor map with a (box_rows x 64) box and the
// 128-byte swizzle.  Returns false with the error message set.
bool make_tmap_f16(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld_elems,
                   int box_rows);

// Encodes a 2-D row-major (rows, cols) tensor map of 2- or 4-byte elements with a box of (box_rows x 64
// BYTES) and the 64-byte swizzle: the layout of the per-warp transposition buffers (32 rows of 64 bytes,
// 16-byte piece p of row r at r * 64 + ((p ^ ((r >> 1) & 3)) << 4)).
bool make_tmap_rows64(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t cols,
                      int64_t ld_elems, int box_rows);
// The same with rows of row_bytes = 64 or 128 bytes (64- / 128-byte swizzle), or any other multiple of 16 (dense rows, no swizzle).
bool make_tmap_rows(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t cols,
                    int64_t ld_elems, int box_rows, int row_bytes);

// Encodes a 3-D fp16 view (cols, tokens_per_env, n_envs) of a token-row matrix whose env e owns rows
// [e * tokens_per_env, (e + 1) * tokens_per_env): box = (box_cols, box_tokens, box_envs).  box_tokens may
// exceed tokens_per_env (29 -> 32): a load then fills the extra rows with zeros and a store skips them, so
// that every env starts on a 32-row boundary of the shared-memory tile.  row_bytes = box_cols * 2 selects the
// swizzle as in make_tmap_rows (128: 128-byte swizzle, 64: 64-byte, otherwise none).
bool make_tmap_env3d(CUtensorMap* map, const void* base, int64_t n_envs, int tokens_per_env, int64_t cols,
                     int64_t ld_elems, int box_cols, int box_tokens, int box_envs);

// Address of the current device's status word (nullptr with the error message set on failure).
int* device_status_ptr();
// Reads and clears the current device's status word (synchronises the device); -1 on failure.
int device_status_take();
// Launches a one-CTA kernel whose only thread waits, with a limit of `polls` polls, on an mbarrier
// that nothing ever arrives on: the wait runs out, the kernel records kSelfTestKernel * 16 + 1 in
// the status word and returns.  Exercises the give-up path without hanging or trapping anything.
constexpr int kSelfTestKernel = 15;
int wait_selftest(uint32_t polls, cudaStream_t stream);

}  // namespace bsrl
