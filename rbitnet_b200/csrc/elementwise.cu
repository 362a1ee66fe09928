// Memory-bound kernels of the step: embedding gather, RMSNorm, rotation of q and k
// with the append to the paged cache, SiLU(gate)*up, and row gather.
// All arithmetic is float32 whatever the storage dtype.
#include "rb_common.cuh"

#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

static thread_local char g_error[512];

void rb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

RB_EXPORT const char* rb_last_error() { return g_error; }

bool rb_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RBITNET_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

RB_EXPORT int rb_abi_version() { return 2; }

RB_EXPORT int rb_device_sm_count() { return rb_sm_count(); }

// 1: the library was built with -DRB_CHECKED (cache addresses are checked before they are used).
RB_EXPORT int rb_is_checked_build() {
#ifdef RB_CHECKED
  return 1;
#else
  return 0;
#endif
}

// ---------------------------------------------------------------- embedding
// x[t, :] = table[ids[t], :] * scale as float32 (crates/bitnet-core/src/llama/model.rs:230-232;
// the reference has no multiplier, scale 1.0).
// An id outside [0, V) is refused on the host before the launch; the kernel
// writes zeros for one rather than read outside the table.
template <typename TW>
__global__ void embed_kernel(float* __restrict__ out, const TW* __restrict__ table,
                             const int* __restrict__ ids, int E, int V, float scale) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  // four values per thread and the whole row in flight at once: the rows come from anywhere in a
  // table far larger than L2, and a loop over the row would wait for memory once per turn
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;
  const TW* row = table + (int64_t)(ok ? id : 0) * E;
  float* o = out + (int64_t)t * E;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (j >= E) return;
  if ((E & 3) == 0) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) {
      if constexpr (sizeof(TW) == 4) {
        v = *reinterpret_cast<const float4*>(row + j);
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(row + j);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        v = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
      }
    }
    if (scale != 1.0f) v = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
    *reinterpret_cast<float4*>(o + j) = v;
  } else {
    for (int i = j; i < min(E, j + 4); ++i) o[i] = ok ? rb_to_float<TW>(row[i]) * scale : 0.f;
  }
}

RB_EXPORT int rb_embed(float* out, const void* table, int table_dtype, const int* ids, int T, int E,
                       int V, float scale, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(T > 0 && E > 0 && V > 0, "rb_embed: bad sizes T=%d E=%d V=%d", T, E, V);
  const int threads = 256;
  const dim3 grid(T, (E + threads * 4 - 1) / (threads * 4));
  RB_REQUIRE(grid.y <= 65535, "rb_embed: rows of %d values", E);
  if (table_dtype == RB_F32)
    RB_LAUNCH("embed_kernel", (embed_kernel<float>), grid, threads, 0, stream, out, (const float*)table, ids, E, V, scale);
  else if (table_dtype == RB_BF16)
    RB_LAUNCH("embed_kernel", (embed_kernel<__nv_bfloat16>), grid, threads, 0, stream, out, (const __nv_bfloat16*)table, ids, E, V, scale);
  else
    RB_FAIL("rb_embed: unknown dtype %d", table_dtype);
  RB_CHECK_LAUNCH("rb_embed");
  return 0;
}

// ---------------------------------------------------------------- RMSNorm
// y = x * w / sqrt(mean(x^2) + eps)  (crates/bitnet-core/src/llama/model.rs:93-100).
// x is the float32 residual stream.
template <typename TO> __device__ __forceinline__ void store4(TO* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}

// VEC: the width is a multiple of 4 and rows are read and written four values at a time.
template <typename TO, bool VEC>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                               int E, float eps) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  __shared__ float scratch[33];
  extern __shared__ __align__(16) float row[];  // E floats
  const int t = blockIdx.x;
  const float* xr = x + (int64_t)t * E;
  float ss = 0.f;
  if (VEC) {
    for (int j = threadIdx.x * 4; j < E; j += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(xr + j);
      *reinterpret_cast<float4*>(row + j) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int j = threadIdx.x; j < E; j += blockDim.x) {
      const float v = xr[j];
      row[j] = v;
      ss += v * v;
    }
  }
  ss = rb_block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)E + eps);
  TO* o = out + (int64_t)t * E;
  if (VEC) {
    for (int j = threadIdx.x * 4; j < E; j += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + j);
      const float4 g = *reinterpret_cast<const float4*>(w + j);
      store4<TO>(o + j, v.x * g.x * r, v.y * g.y * r, v.z * g.z * r, v.w * g.w * r);
    }
  } else {
    for (int j = threadIdx.x; j < E; j += blockDim.x) o[j] = rb_from_float<TO>(row[j] * w[j] * r);
  }
}

// Rows of up to 4*NV*blockDim values (a multiple of 4) kept in registers: every load of a row
// is in flight before the first is used, and nothing goes through shared memory.
template <typename TO, int NV>
__global__ void rmsnorm_reg_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                                   int E, float eps) {
  rb_pdl_launch_dependents();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float* xr = x + (int64_t)t * E;
  float4 v[NV], g[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {       // the norm's weights do not depend on the kernel before
    const int j = (threadIdx.x + i * blockDim.x) * 4;
    g[i] = j < E ? *reinterpret_cast<const float4*>(w + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  rb_pdl_wait();
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (threadIdx.x + i * blockDim.x) * 4;
    v[i] = j < E ? *reinterpret_cast<const float4*>(xr + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  ss = rb_block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)E + eps);
  TO* o = out + (int64_t)t * E;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (threadIdx.x + i * blockDim.x) * 4;
    if (j < E) store4<TO>(o + j, v[i].x * g[i].x * r, v[i].y * g[i].y * r, v[i].z * g[i].z * r, v[i].w * g[i].w * r);
  }
}

template <typename TO>
static int launch_rmsnorm_reg(TO* out, const float* x, const float* w, int T, int E, float eps, cudaStream_t stream) {
  const int threads = E <= 1024 ? 128 : (E <= 4096 ? 256 : 1024);
  const int nv = (E / 4 + threads - 1) / threads;
  switch (nv) {
    case 1: RB_LAUNCH("rmsnorm_reg_kernel", (rmsnorm_reg_kernel<TO, 1>), T, threads, 0, stream, out, x, w, E, eps); break;
    case 2: RB_LAUNCH("rmsnorm_reg_kernel", (rmsnorm_reg_kernel<TO, 2>), T, threads, 0, stream, out, x, w, E, eps); break;
    case 3: RB_LAUNCH("rmsnorm_reg_kernel", (rmsnorm_reg_kernel<TO, 3>), T, threads, 0, stream, out, x, w, E, eps); break;
    default: RB_LAUNCH("rmsnorm_reg_kernel", (rmsnorm_reg_kernel<TO, 4>), T, threads, 0, stream, out, x, w, E, eps); break;
  }
  RB_CHECK_LAUNCH("rb_rmsnorm");
  return 0;
}

template <typename TO, bool VEC>
static int launch_rmsnorm(TO* out, const float* x, const float* w, int T, int E, float eps, cudaStream_t stream) {
  const int per = VEC ? 4 : 1;
  int threads = 128;
  while (threads < 1024 && threads * per * 2 <= E) threads *= 2;     // about two loads per thread
  const size_t smem = (size_t)E * sizeof(float);
  if (smem > 48 * 1024)
    RB_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<TO, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RB_LAUNCH("rmsnorm_kernel", (rmsnorm_kernel<TO, VEC>), T, threads, smem, stream, out, x, w, E, eps);
  RB_CHECK_LAUNCH("rb_rmsnorm");
  return 0;
}

RB_EXPORT int rb_rmsnorm(void* out, int out_dtype, const float* x, const float* w, int T, int E, float eps,
                         cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(T > 0 && E > 0, "rb_rmsnorm: bad sizes T=%d E=%d", T, E);
  RB_REQUIRE((size_t)E * 4 <= 200 * 1024, "rb_rmsnorm: width %d exceeds the %d floats one block can hold",
             E, 200 * 1024 / 4);
  const bool vec = E % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                   ((uintptr_t)out % 16 == 0);
  if (vec && E <= 16384) {
    if (out_dtype == RB_F32)
      return launch_rmsnorm_reg<float>((float*)out, x, w, T, E, eps, stream);
    if (out_dtype == RB_BF16)
      return launch_rmsnorm_reg<__nv_bfloat16>((__nv_bfloat16*)out, x, w, T, E, eps, stream);
  }
  if (out_dtype == RB_F32)
    return vec ? launch_rmsnorm<float, true>((float*)out, x, w, T, E, eps, stream)
               : launch_rmsnorm<float, false>((float*)out, x, w, T, E, eps, stream);
  if (out_dtype == RB_BF16)
    return vec ? launch_rmsnorm<__nv_bfloat16, true>((__nv_bfloat16*)out, x, w, T, E, eps, stream)
               : launch_rmsnorm<__nv_bfloat16, false>((__nv_bfloat16*)out, x, w, T, E, eps, stream);
  RB_FAIL("rb_rmsnorm: unknown dtype %d", out_dtype);
}

// ---------------------------------------------------------------- rotation + cache append
// For every new token: rotate each q head and each k head by the token's
// position (angle = pos * inv_freq[i], float32; pairs (2i,2i+1) when
// `interleaved`, else (i, i+D/2)), write q to q_out[T,H,D], the rotated k and
// the raw v to the token's place in the paged cache.
// crates/bitnet-core/src/llama/model.rs:122-136 (rotation), :242-257 (append).
// `qkv` rows hold [H*D | Kh*D | Kh*D]; with write_kv == 0 only q is read (a
// layer that reads another layer's cache).  Only the first rot_dim values of a head are
// rotated (pairs (2i,2i+1) or (i, i+rot_dim/2) among them); the rest pass unchanged.
template <typename T>
__global__ void rotate_append_kernel(T* __restrict__ q_out, const T* __restrict__ qkv, int64_t qkv_stride,
                                     const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_slot, RbPagedLayer cache, int H, int write_kv,
                                     int interleaved, int heads_per_block, int rot_dim) {
  rb_pdl_launch_dependents();
  const int t = blockIdx.x;
  const int D = cache.head_dim, Kh = cache.n_kv_heads;
  const int pos = tok_pos[t];
  const int slot = tok_slot[t];
  rb_pdl_wait();     // positions and slots were written before the step began; qkv comes from the kernel before
  const T* row = qkv + (int64_t)t * qkv_stride;
  auto value = [&](int64_t i) { return rb_to_float<T>(row[i]); };
  const int half = D / 2;
  const int n_rot_heads = H + (write_kv ? Kh : 0);
  const int n_heads = n_rot_heads + (write_kv ? Kh : 0);        // rotated heads, then the v heads
  const int h0 = blockIdx.y * heads_per_block, h1 = min(n_heads, h0 + heads_per_block);
  T* kdst = (T*)cache.k;
  T* vdst = (T*)cache.v;
  // one thread per pair of values: a rotated pair of a q or k head, or two neighbours of a v head
  for (int idx = threadIdx.x; idx < (h1 - h0) * half; idx += blockDim.x) {
    const int head = h0 + idx / half, i = idx % half;
    const int64_t src = (int64_t)head * D;  // q heads, k heads, v heads are contiguous in a row
    if (head >= n_rot_heads) {
      T* dst = vdst + rb_page_offset(cache, slot, pos, head - n_rot_heads);
      dst[2 * i] = rb_from_float<T>(value(src + 2 * i));
      dst[2 * i + 1] = rb_from_float<T>(value(src + 2 * i + 1));
      continue;
    }
    T* dst = head < H ? q_out + ((int64_t)t * H + head) * D : kdst + rb_page_offset(cache, slot, pos, head - H);
    const int rhalf = rot_dim / 2;
    if (i >= rhalf) {           // behind the rotated prefix: two neighbours, as they are
      const int a = rot_dim + 2 * (i - rhalf);
      dst[a] = rb_from_float<T>(value(src + a));
      dst[a + 1] = rb_from_float<T>(value(src + a + 1));
      continue;
    }
    int a, b;
    if (interleaved) { a = 2 * i; b = 2 * i + 1; } else { a = i; b = i + rhalf; }
    const float x0 = value(src + a);
    const float x1 = value(src + b);
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    const float y0 = x0 * cs - x1 * sn;
    const float y1 = x0 * sn + x1 * cs;
    dst[a] = rb_from_float<T>(y0);
    dst[b] = rb_from_float<T>(y1);
  }
}

// Many tokens, bfloat16 in and out, head_dim a multiple of 16: one block per token.  A thread owns
// eight rotation pairs (the same eight in every head), computes their sines and cosines once,
// and walks over the heads with 16-byte loads and stores; values are copied 16 bytes at a time.
constexpr int ROWS_MAX_PAIRS = 256;      // head sizes up to 512 take the many-token kernel
__global__ void __launch_bounds__(1024) rotate_append_rows_kernel(
    __nv_bfloat16* __restrict__ q_out, const __nv_bfloat16* __restrict__ qkv, int64_t qkv_stride,
    const float* __restrict__ inv_freq, const int* __restrict__ tok_pos, const int* __restrict__ tok_slot,
    RbPagedLayer cache, int H, int write_kv, int interleaved) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t = blockIdx.x;
  const int D = cache.head_dim, Kh = cache.n_kv_heads;
  const int pos = tok_pos[t], slot = tok_slot[t];
  const __nv_bfloat16* row = qkv + (int64_t)t * qkv_stride;
  const int groups = D / 16;                       // groups of eight pairs per head
  const int lanes = blockDim.x / groups;           // threads that share a group walk different heads
  const int grp = threadIdx.x % groups, lane = threadIdx.x / groups;
  const int n_rot = H + (write_kv ? Kh : 0);
  __nv_bfloat16* kdst = (__nv_bfloat16*)cache.k;
  __nv_bfloat16* vdst = (__nv_bfloat16*)cache.v;
  // element offsets of the two 16-byte pieces this thread rotates in every head
  const int off_a = interleaved ? grp * 16 : grp * 8;
  const int off_b = interleaved ? grp * 16 + 8 : D / 2 + grp * 8;
  // the first head's values and the value rows are asked for before anything else, so that the loads
  // run while the sines and cosines are made (with one thread per head and group that is all of them)
  const bool active = lane < lanes && lane < n_rot;
  uint4 va = make_uint4(0, 0, 0, 0), vb = va, vv = va;
  if (active) {
    va = *reinterpret_cast<const uint4*>(row + (int64_t)lane * D + off_a);
    vb = *reinterpret_cast<const uint4*>(row + (int64_t)lane * D + off_b);
  }
  const int per_head = D / 8;
  const bool copies = write_kv && (int)threadIdx.x < Kh * per_head;
  if (copies) vv = *reinterpret_cast<const uint4*>(row + (int64_t)(H + Kh) * D + (int64_t)threadIdx.x * 8);
  // the token's D/2 sines and cosines, once per block
  __shared__ float s_sn[ROWS_MAX_PAIRS], s_cs[ROWS_MAX_PAIRS];
  for (int i = threadIdx.x; i < D / 2; i += blockDim.x) sincosf((float)pos * inv_freq[i], &s_sn[i], &s_cs[i]);
  __syncthreads();
  if (active) {
    float sn[8], cs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sn[j] = s_sn[grp * 8 + j]; cs[j] = s_cs[grp * 8 + j]; }
    for (int head = lane; head < n_rot; head += lanes) {
      if (head != lane) {
        va = *reinterpret_cast<const uint4*>(row + (int64_t)head * D + off_a);
        vb = *reinterpret_cast<const uint4*>(row + (int64_t)head * D + off_b);
      }
      __nv_bfloat16* ea = reinterpret_cast<__nv_bfloat16*>(&va);
      __nv_bfloat16* eb = reinterpret_cast<__nv_bfloat16*>(&vb);
      if (interleaved) {
        // pairs (2i, 2i+1): pairs 0..3 lie in va, 4..7 in vb
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_bfloat16* e = j < 4 ? ea : eb;
          const int o = (j & 3) * 2;
          const float x0 = __bfloat162float(e[o]), x1 = __bfloat162float(e[o + 1]);
          e[o] = __float2bfloat16_rn(x0 * cs[j] - x1 * sn[j]);
          e[o + 1] = __float2bfloat16_rn(x0 * sn[j] + x1 * cs[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float x0 = __bfloat162float(ea[j]), x1 = __bfloat162float(eb[j]);
          ea[j] = __float2bfloat16_rn(x0 * cs[j] - x1 * sn[j]);
          eb[j] = __float2bfloat16_rn(x0 * sn[j] + x1 * cs[j]);
        }
      }
      __nv_bfloat16* dst = head < H ? q_out + ((int64_t)t * H + head) * D
                                    : kdst + rb_page_offset(cache, slot, pos, head - H);
      *reinterpret_cast<uint4*>(dst + off_a) = va;
      *reinterpret_cast<uint4*>(dst + off_b) = vb;
    }
  }
  if (write_kv) {
    const __nv_bfloat16* vsrc = row + (int64_t)(H + Kh) * D;
    for (int idx = threadIdx.x; idx < Kh * per_head; idx += blockDim.x) {
      const int kvh = idx / per_head, c = idx % per_head;
      if (idx != (int)threadIdx.x) vv = *reinterpret_cast<const uint4*>(vsrc + (int64_t)kvh * D + c * 8);
      *reinterpret_cast<uint4*>(vdst + rb_page_offset(cache, slot, pos, kvh) + c * 8) = vv;
    }
  }
}

// dtype: the type of qkv, of q_out and of the cache.
RB_EXPORT int rb_rotate_append(void* q_out, const void* qkv, int64_t qkv_stride, int dtype,
                               const float* inv_freq, const int* tok_pos, const int* tok_slot, void* cache_k,
                               void* cache_v, const int* page_table, int max_pages, int page_size, int T, int H,
                               int Kh, int D, int write_kv, int rot_dim, int interleaved, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(D % 2 == 0 && D > 0, "rb_rotate_append: head_dim %d must be even", D);
  RB_REQUIRE(rot_dim >= 0 && rot_dim <= D && rot_dim % 2 == 0,
             "rb_rotate_append: the rotated prefix %d must be even and at most the head size %d", rot_dim, D);
  RB_REQUIRE(H > 0 && Kh >= 0 && page_size > 0, "rb_rotate_append: bad sizes H=%d Kh=%d page=%d", H, Kh, page_size);
  RbPagedLayer c{cache_k, cache_v, page_table, max_pages, page_size, Kh, D};
  const int threads = 256;
  // few tokens: spread a token's heads over several blocks so that enough blocks run
  const int n_heads = H + (write_kv ? 2 * Kh : 0);
  int by = T >= 128 ? 1 : (128 + T - 1) / T;
  if (by > n_heads) by = n_heads;
  const int hpb = (n_heads + by - 1) / by;
  const dim3 grid(T, (n_heads + hpb - 1) / hpb);
  if (dtype == RB_BF16 && T >= 32 && rot_dim == D && D % 16 == 0 && D <= 2 * ROWS_MAX_PAIRS &&
      qkv_stride % 8 == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
      ((uintptr_t)cache_k % 16 == 0) && ((uintptr_t)cache_v % 16 == 0)) {
    // one thread per (rotated head, group of eight pairs) where a block can hold them: one pass over the heads
    const int items = (H + (write_kv ? Kh : 0)) * (D / 16);
    const int rows_threads = items >= 1024 ? 1024 : (items < 128 ? 128 : (items + 31) / 32 * 32);
    RB_LAUNCH("rotate_append_rows_kernel", (rotate_append_rows_kernel), T, rows_threads, 0, stream, (__nv_bfloat16*)q_out,
              (const __nv_bfloat16*)qkv, qkv_stride, inv_freq, tok_pos, tok_slot, c, H, write_kv, interleaved);
    return 0;
  }
  if (dtype == RB_F32)
    RB_LAUNCH("rotate_append_kernel", (rotate_append_kernel<float>), grid, threads, 0, stream, (float*)q_out, (const float*)qkv, qkv_stride, inv_freq, tok_pos, tok_slot, c, H, write_kv, interleaved, hpb, rot_dim);
  else if (dtype == RB_BF16)
    RB_LAUNCH("rotate_append_kernel", (rotate_append_kernel<__nv_bfloat16>), grid, threads, 0, stream, (__nv_bfloat16*)q_out, (const __nv_bfloat16*)qkv, qkv_stride, inv_freq, tok_pos, tok_slot, c, H, write_kv, interleaved, hpb, rot_dim);
  else
    RB_FAIL("rb_rotate_append: unknown dtype %d", dtype);
  RB_CHECK_LAUNCH("rb_rotate_append");
  return 0;
}

// ---------------------------------------------------------------- SiLU(gate) * up
// out[t, j] = silu(gate[t, j]) * up[t, j], silu(v) = v / (1 + exp(-v)), in float32.
// crates/bitnet-core/src/llama/model.rs:116-120, 297-302
// block == 0: a row of gu is [gate (F) | up (F)].  block == B > 0: it is made of groups of 2B
// values, B of gate followed by the B of up for the same features (the row order the tensor-core
// gated product wants of its weights); `ld` is the row length of gu.
template <typename T, typename TI>
__global__ void silu_mul_kernel(T* __restrict__ out, const TI* __restrict__ gu, int64_t n, int F, int64_t ld, int block) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / F;
    const int j = (int)(i % F);
    const int64_t at_g = block > 0 ? (int64_t)(j / block) * 2 * block + j % block : j;
    const int64_t at_u = block > 0 ? at_g + block : (int64_t)F + j;
    const float g = rb_to_float<TI>(gu[t * ld + at_g]);
    const float u = rb_to_float<TI>(gu[t * ld + at_u]);
    out[i] = rb_from_float<T>(g / (1.0f + expf(-g)) * u);
  }
}

// in_dtype: dtype of gate_up (the output dtype, or RB_F32 for a bfloat16 output).
RB_EXPORT int rb_silu_mul(void* out, const void* gate_up, int dtype, int in_dtype, int T, int F, int64_t ld, int block,
                          cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(block >= 0 && (block == 0 ? ld >= 2 * (int64_t)F : ld >= ((int64_t)(F + block - 1) / block) * 2 * block),
             "rb_silu_mul: rows of %lld values do not hold %d features in blocks of %d", (long long)ld, F, block);
  const int64_t n = (int64_t)T * F;
  const int threads = 256;
  const int64_t most = (int64_t)rb_sm_count() * 16;
  const int blocks = (int)((n + threads - 1) / threads < most ? (n + threads - 1) / threads : most);
  if (dtype == RB_F32 && in_dtype == RB_F32)
    RB_LAUNCH("silu_mul_kernel", (silu_mul_kernel<float, float>), blocks, threads, 0, stream, (float*)out, (const float*)gate_up, n, F, ld, block);
  else if (dtype == RB_BF16 && in_dtype == RB_BF16)
    RB_LAUNCH("silu_mul_kernel", (silu_mul_kernel<__nv_bfloat16, __nv_bfloat16>), blocks, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, n, F, ld, block);
  else if (dtype == RB_BF16 && in_dtype == RB_F32)
    RB_LAUNCH("silu_mul_kernel", (silu_mul_kernel<__nv_bfloat16, float>), blocks, threads, 0, stream, (__nv_bfloat16*)out, (const float*)gate_up, n, F, ld, block);
  else
    RB_FAIL("rb_silu_mul: unsupported dtypes %d <- %d", dtype, in_dtype);
  return 0;
}

// ---------------------------------------------------------------- row gather (float32 residual rows)
__global__ void gather_rows_kernel(float* __restrict__ out, const float* __restrict__ x,
                                   const int* __restrict__ rows, int E) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  // one element (or one group of four) per thread: the copies of a row are all in flight together
  const int r = blockIdx.x;
  const float* src = x + (int64_t)rows[r] * E;
  float* dst = out + (int64_t)r * E;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if ((E & 3) == 0) {
    if (j < E) *reinterpret_cast<float4*>(dst + j) = *reinterpret_cast<const float4*>(src + j);
  } else {
    for (int i = j; i < min(E, j + 4); ++i) dst[i] = src[i];
  }
}

RB_EXPORT int rb_gather_rows(float* out, const float* x, const int* rows, int R, int E, cudaStream_t stream) {
  if (R == 0) return 0;
  RB_REQUIRE(R <= 2147483647 && (E + 1023) / 1024 <= 65535, "rb_gather_rows: %d rows of %d", R, E);
  RB_LAUNCH("gather_rows_kernel", (gather_rows_kernel), dim3(R, (E + 1023) / 1024), 256, 0, stream, out, x, rows, E);
  RB_CHECK_LAUNCH("rb_gather_rows");
  return 0;
}

// ---------------------------------------------------------------- decode bookkeeping on the device
// After a decode step has sampled: the sampled ids become the next step's tokens and every
// position moves on by one, so that steps can follow one another without the host.  Only the first
// *n_live rows move (n_live null: all B): rows behind them belong to the padding sequence, which
// rewrites its position 0 at every step.
__global__ void decode_advance_kernel(int* __restrict__ token_ids, int* __restrict__ tok_pos,
                                      const int* __restrict__ sampled, int B, const int* __restrict__ n_live,
                                      const int* flag_a, const int* flag_b, int* __restrict__ flag_out) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int live = n_live != nullptr ? *n_live : B;
  if (i < B && i < live) {
    token_ids[i] = sampled[i];
    tok_pos[i] += 1;
  }
  // the error words of the kernels that wait on barriers travel with the step's results
  if (i == 0 && flag_out != nullptr) {
    const int a = flag_a != nullptr ? *flag_a : 0, b = flag_b != nullptr ? *flag_b : 0;
    *flag_out = a != 0 ? a : b;
  }
}

RB_EXPORT int rb_decode_advance(int* token_ids, int* tok_pos, const int* sampled, int B, const int* n_live,
                                const int* flag_a, const int* flag_b, int* flag_out, cudaStream_t stream) {
  if (B == 0) return 0;
  RB_LAUNCH("decode_advance_kernel", (decode_advance_kernel), (B + 127) / 128, 128, 0, stream, token_ids, tok_pos, sampled, B,
            n_live, flag_a, flag_b, flag_out);
  RB_CHECK_LAUNCH("rb_decode_advance");
  return 0;
}

RB_CHECK_READER(elementwise)
