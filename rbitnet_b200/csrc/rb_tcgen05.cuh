// Device-side wrappers of the sm_100a instructions the tensor-core kernels share: mbarrier with
// bounded waits, TMA tile loads, tcgen05 MMA / commit / fences / tensor-memory loads and stores,
// and the shared-memory operand descriptor of the 128-byte swizzle.
#pragma once

#include "rb_common.cuh"

#include <cuda.h>

// The device word that a kernel sets when one of its bounded waits ran out (0: none).  Each
// source file that includes this header has its own copy; rb_read_error_flag() reads them all.
static __device__ int g_error_flag = 0;

static inline int rb_file_error_flag(int* value, int reset) {
  int v = 0;
  RB_CUDA(cudaMemcpyFromSymbol(&v, g_error_flag, sizeof(int)));
  if (reset && v != 0) {
    int z = 0;
    RB_CUDA(cudaMemcpyToSymbol(g_error_flag, &z, sizeof(int)));
  }
  *value = v;
  return 0;
}

static inline int rb_file_set_error_flag(int code) {
  RB_CUDA(cudaMemcpyToSymbol(g_error_flag, &code, sizeof(int)));
  return 0;
}

// Device address of this file's error word (for a kernel that reports it with a step's results).
static inline int rb_file_error_flag_address(int** out) {
  void* p = nullptr;
  RB_CUDA(cudaGetSymbolAddress(&p, g_error_flag));
  *out = (int*)p;
  return 0;
}

// Tensor map of a row-major bfloat16 matrix [rows, cols] (cols contiguous, row stride ld elements),
// box [box_rows, 64], 128-byte swizzle, zero fill outside; cached by its arguments.
int rb_get_tensor_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int64_t ld, int box_rows);
// The same for an output: float32 (elem_bytes 4) or bfloat16 (2), box [box_rows, box_cols], no swizzle.
int rb_get_output_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int64_t ld, int box_rows, int box_cols,
                      int elem_bytes);


// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// One poll of the barrier.  The thread may be parked by the hardware until the phase completes
// or about `hint_ns` have passed, so a waiting thread does not fill issue slots with polls.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns = 20000u) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false (and the error word set to `code`) after `limit_ns`, about 2 s in the kernels.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code,
                                          uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 1024; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) {
      atomicCAS(&g_error_flag, 0, code);
      return false;
    }
  }
}
// Bounded wait for a word in global memory to reach `value` (another CTA of the same launch stores
// it with release): false, and the error word set to `code`, after `limit_ns`.
__device__ __forceinline__ bool wait_for_count(const int* word, int value, int code, uint64_t limit_ns = 2000000000ull) {
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
      int v;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
      if (v == value) return true;
      __nanosleep(64);
    }
    if (global_timer_ns() - t0 > limit_ns) {
      atomicCAS(&g_error_flag, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// A box of shared memory to global memory through a tensor map (rows outside the tensor are
// dropped); `add`: added to what is there, in the tensor's own type, instead of stored.  Bulk-group
// completion: commit after issuing, wait before the shared memory is written again.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y, bool add) {
  if (add)
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(src)), "r"(x), "r"(y)
                 : "memory");
  else
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's bulk groups have read their shared memory
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all of this thread's bulk groups are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused with a swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                    // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                    // 128-byte swizzle
  return d;
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }


__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// General form of the instruction descriptor: bfloat16 operands, float32 accumulator;
// a_mn / b_mn: the operand's M (or N) dimension is the contiguous one in shared memory.
__host__ __device__ constexpr uint32_t make_idesc_mn(int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
