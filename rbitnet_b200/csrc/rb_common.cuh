// Shared helpers of the rbitnet_b200 kernels (sm_100a only).
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes
// and the stream to launch on, and returns 0 or a negative code; the message
// of the last failure of the calling thread is read with rb_last_error().
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define RB_EXPORT extern "C" __attribute__((visibility("default")))

enum RbDtype { RB_F32 = 0, RB_BF16 = 1 };

void rb_set_error(const char* fmt, ...);

#define RB_FAIL(...)                 \
  do {                               \
    rb_set_error(__VA_ARGS__);       \
    return -1;                       \
  } while (0)

#define RB_REQUIRE(cond, ...)        \
  do {                               \
    if (!(cond)) RB_FAIL(__VA_ARGS__); \
  } while (0)

#define RB_CHECK_LAUNCH(name)                                                     \
  do {                                                                            \
    cudaError_t e__ = cudaGetLastError();                                         \
    if (e__ != cudaSuccess) RB_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
  } while (0)

#define RB_CUDA(call)                                                             \
  do {                                                                            \
    cudaError_t e__ = (call);                                                     \
    if (e__ != cudaSuccess) RB_FAIL("%s failed: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of the library is launched with the attribute that lets it start while the
// kernel before it in the stream is still running.  A kernel therefore calls rb_pdl_wait()
// before its first access to global memory (after the wait, everything earlier in the stream
// has completed and is visible), and rb_pdl_launch_dependents() as early as it can, so that
// the next kernel's launch and set-up overlap this kernel's work.  Inside a captured graph the
// same launches become programmatic edges.
__device__ __forceinline__ void rb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void rb_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool rb_pdl_enabled();   // RBITNET_PDL=0 in the environment turns the launch attribute off

template <typename... KArgs, typename... Args>
inline cudaError_t rb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = rb_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define RB_LAUNCH(name, kernel, grid, block, smem, stream, ...)                              \
  do {                                                                                       \
    cudaError_t e__ = rb_launch(kernel, grid, block, smem, stream, __VA_ARGS__);             \
    if (e__ != cudaSuccess) RB_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// ---------------------------------------------------------------- per-device facts and set-up
constexpr int RB_MAX_DEVICES = 64;

// Number of SMs of the current device (asked once per device).
inline int rb_sm_count() {
  static int n[RB_MAX_DEVICES] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= RB_MAX_DEVICES) dev = 0;
  if (n[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

// Set-up that has to happen once per device (a kernel's shared-memory attribute belongs to the
// device that was current when it was set): true the first time it is asked for the current device.
struct RbOncePerDevice {
  bool done[RB_MAX_DEVICES] = {false};
  bool first() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= RB_MAX_DEVICES) return true;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
  }
};

// ---------------------------------------------------------------- scalar conversions
template <typename T> __device__ __forceinline__ float rb_to_float(T v);
template <> __device__ __forceinline__ float rb_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float rb_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T rb_from_float(float v);
template <> __device__ __forceinline__ float rb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 rb_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------- reductions
__device__ __forceinline__ float rb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float rb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 33 floats of shared
// memory.  All threads get the result.
__device__ __forceinline__ float rb_block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = rb_warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = rb_warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float rb_block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = rb_warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = rb_warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---------------------------------------------------------------- paged cache addressing
// One layer's keys (or values) live in pages of `page_size` positions:
//   base[page][kv_head][position in page][d]
// and a sequence's pages are listed in its row of the page table.
struct RbPagedLayer {
  void* k;                 // keys of this layer
  void* v;                 // values of this layer
  const int* page_table;   // [n_slots, max_pages]
  int max_pages;           // row length of the page table
  int page_size;           // positions per page
  int n_kv_heads;
  int head_dim;
};

// ---------------------------------------------------------------- the checked build
// With -DRB_CHECKED (RBITNET_CHECKED=1 when the library is built) every cache address that goes
// through rb_page_offset is checked first: a slot, position or kv head outside what the layer holds
// is recorded in a device word (code 21, then the slot, the position and the kv head) and the
// access goes to offset 0 instead of outside the cache.  Each source file has its own word and
// exports a reader for it (RB_CHECK_READER); the host asks them all after a step.
#ifdef RB_CHECKED
static __device__ int g_check_word[4] = {0, 0, 0, 0};
#define RB_CHECK_READER(tu)                                                        \
  RB_EXPORT int rb_check_word_##tu(int* out4, int reset) {                         \
    RB_CUDA(cudaMemcpyFromSymbol(out4, g_check_word, 4 * sizeof(int)));            \
    if (reset && out4[0] != 0) {                                                   \
      int z[4] = {0, 0, 0, 0};                                                     \
      RB_CUDA(cudaMemcpyToSymbol(g_check_word, z, 4 * sizeof(int)));               \
    }                                                                              \
    return 0;                                                                      \
  }
#else
#define RB_CHECK_READER(tu)                                                        \
  RB_EXPORT int rb_check_word_##tu(int* out4, int reset) {                         \
    (void)reset;                                                                   \
    out4[0] = out4[1] = out4[2] = out4[3] = 0;                                     \
    return 0;                                                                      \
  }
#endif

__device__ __forceinline__ int64_t rb_page_offset(const RbPagedLayer& c, int slot, int pos, int kvh) {
#ifdef RB_CHECKED
  if (slot < 0 || pos < 0 || pos / c.page_size >= c.max_pages || kvh < 0 || kvh >= c.n_kv_heads) {
    if (atomicCAS(&g_check_word[0], 0, 21) == 0) {
      g_check_word[1] = slot;
      g_check_word[2] = pos;
      g_check_word[3] = kvh;
    }
    return 0;
  }
#endif
  const int page = c.page_table[(int64_t)slot * c.max_pages + pos / c.page_size];
  return (((int64_t)page * c.n_kv_heads + kvh) * c.page_size + pos % c.page_size) * c.head_dim;
}
