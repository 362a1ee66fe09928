// Plain attention over the paged cache: one warp per (token, query head), keys
// visited one by one in ascending position with a running max and sum
// (float32).  It serves the true 32-bit path, and any shape the tiled kernels
// refuse.  Because each (token, head) is reduced alone and in a fixed order,
// its result is bit-identical however the tokens were cut into steps or
// batched.
//
// Token t at position p of its sequence attends keys max(0, p-window+1)..p of
// its own slot; query head h reads kv head h / (H/Kh); the score is
// (q.k) * scale with the scale applied to the finished dot product; softmax is
// max-subtracted.  crates/bitnet-core/src/llama/model.rs:260-289, :102-114
#include "rb_common.cuh"

namespace {

template <typename T, int EPL>
__global__ void __launch_bounds__(128) attn_simple_kernel(T* __restrict__ out, const T* __restrict__ q,
                                                         RbPagedLayer cache, const int* __restrict__ tok_pos,
                                                         const int* __restrict__ tok_slot, int n_tokens, int H,
                                                         float scale, int window) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * 4 + warp;
  if (w >= (int64_t)n_tokens * H) return;
  const int t = (int)(w / H), h = (int)(w % H);
  const int D = cache.head_dim;
  const int kvh = h / (H / cache.n_kv_heads);
  const int pos = tok_pos[t], slot = tok_slot[t];
  const T* qp = q + ((int64_t)t * H + h) * D;
  const T* Kb = (const T*)cache.k;
  const T* Vb = (const T*)cache.v;

  float qr[EPL], acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int d = lane + 32 * e;
    qr[e] = d < D ? rb_to_float<T>(qp[d]) : 0.f;
    acc[e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  for (int p = lo; p <= pos; ++p) {
    const int64_t off = rb_page_offset(cache, slot, p, kvh);
    float part = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = lane + 32 * e;
      if (d < D) part = fmaf(qr[e], rb_to_float<T>(Kb[off + d]), part);
    }
    const float s = rb_warp_sum(part) * scale;
    const float mn = fmaxf(m, s);
    const float corr = expf(m - mn);   // exp(-inf) = 0 on the first key
    const float pe = expf(s - mn);
    l = l * corr + pe;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = lane + 32 * e;
      if (d < D) acc[e] = acc[e] * corr + pe * rb_to_float<T>(Vb[off + d]);
    }
    m = mn;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* op = out + ((int64_t)t * H + h) * D;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int d = lane + 32 * e;
    if (d < D) op[d] = rb_from_float<T>(acc[e] * inv);
  }
}

template <typename T>
int launch(T* out, const T* q, RbPagedLayer c, const int* tok_pos, const int* tok_slot, int n_tokens, int H,
           float scale, int window, cudaStream_t stream) {
  const int64_t warps = (int64_t)n_tokens * H;
  const int blocks = (int)((warps + 3) / 4);
  const int epl = (c.head_dim + 31) / 32;
#define CASE(E) \
  case E: RB_LAUNCH("attn_simple_kernel", (attn_simple_kernel<T, E>), blocks, 128, 0, stream, out, q, c, tok_pos, tok_slot, n_tokens, H, scale, window); break;
  switch (epl) {
    CASE(1) CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7) CASE(8)
    default: RB_FAIL("rb_attention_simple: head_dim %d exceeds 256", c.head_dim);
  }
#undef CASE
  RB_CHECK_LAUNCH("rb_attention_simple");
  return 0;
}

}  // namespace

RB_EXPORT int rb_attention_simple(void* out, const void* q, int dtype, const void* cache_k, const void* cache_v,
                                  const int* page_table, int max_pages, int page_size, const int* tok_pos,
                                  const int* tok_slot, int n_tokens, int H, int Kh, int D, float scale,
                                  int window, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  RB_REQUIRE(H > 0 && Kh > 0 && H % Kh == 0, "rb_attention_simple: heads %d not a multiple of kv heads %d", H, Kh);
  RB_REQUIRE(D > 0 && D <= 256, "rb_attention_simple: head_dim %d must be in 1..256", D);
  RbPagedLayer c{(void*)cache_k, (void*)cache_v, page_table, max_pages, page_size, Kh, D};
  if (dtype == RB_F32)
    return launch<float>((float*)out, (const float*)q, c, tok_pos, tok_slot, n_tokens, H, scale, window, stream);
  if (dtype == RB_BF16)
    return launch<__nv_bfloat16>((__nv_bfloat16*)out, (const __nv_bfloat16*)q, c, tok_pos, tok_slot, n_tokens, H,
                                 scale, window, stream);
  RB_FAIL("rb_attention_simple: unknown dtype %d", dtype);
}

RB_CHECK_READER(attention_simple)
