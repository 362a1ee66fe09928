// Next-token choice on the device, one block per row of logits.
//
// temperature <= 0: the index of the largest logit, NaN counted as -inf, the
// LOWEST index among equal maxima (the reference's iterator keeps the last of
// equal maxima, crates/bitnet-core/src/llama/runtime.rs:82-93; the lowest is
// this library's documented, batch-independent rule).
// temperature > 0: z/T, max-subtracted exp, total S, r = u*S, the first index
// whose running sum reaches r, else the last index
// (crates/bitnet-core/src/llama/runtime.rs:94-106).  u in [0,1) comes from the
// host, one per row, so that the draw is a function of (seed, request, step)
// and of nothing else.
#include "rb_common.cuh"

namespace {

constexpr int THREADS = 1024;

__global__ void __launch_bounds__(THREADS) sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                        int64_t row_stride, int V,
                                                        const float* __restrict__ temperature,
                                                        const float* __restrict__ uniform) {
  __shared__ float scratch[33];
  __shared__ float chunk_sum[THREADS];
  __shared__ int s_best;
  const int r = blockIdx.x;
  const float* z = logits + (int64_t)r * row_stride;
  const float temp = temperature[r];
  const int tid = threadIdx.x;

  // max (NaN counts as -inf)
  float m = -INFINITY;
  for (int i = tid; i < V; i += THREADS) {
    const float v = z[i];
    if (!(v != v)) m = fmaxf(m, v);
  }
  m = rb_block_max(m, scratch);

  if (!(temp > 0.f)) {
    if (tid == 0) s_best = V;  // becomes the lowest index holding the max
    __syncthreads();
    int best = V;
    for (int i = tid; i < V; i += THREADS) {
      float v = z[i];
      if (v != v) v = -INFINITY;
      if (v == m) { best = i; break; }
    }
    atomicMin(&s_best, best);
    __syncthreads();
    if (tid == 0) out[r] = s_best < V ? s_best : 0;
    return;
  }

  // each thread owns a contiguous chunk so that running sums follow index order
  const int per = (V + THREADS - 1) / THREADS;
  const int lo = min(V, tid * per), hi = min(V, lo + per);
  const float inv_t = 1.0f / temp;
  float local = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float v = z[i];
    if (!(v != v)) local += expf((v - m) * inv_t);
  }
  chunk_sum[tid] = local;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int i = 0; i < THREADS; ++i) total += chunk_sum[i];
    const float target = uniform[r] * total;
    // find the chunk, then walk it
    float c = 0.f;
    int chunk = THREADS - 1;
    for (int i = 0; i < THREADS; ++i) {
      if (c + chunk_sum[i] >= target) { chunk = i; break; }
      c += chunk_sum[i];
    }
    const int clo = min(V, chunk * per), chi = min(V, clo + per);
    int pick = V - 1;
    for (int i = clo; i < chi; ++i) {
      const float v = z[i];
      if (!(v != v)) c += expf((v - m) * inv_t);
      if (c >= target) { pick = i; break; }
    }
    if (pick == V - 1 && chi < V) {
      // rounding left the target just past this chunk: go on in index order
      for (int i = chi; i < V; ++i) {
        const float v = z[i];
        if (!(v != v)) c += expf((v - m) * inv_t);
        if (c >= target) { pick = i; break; }
      }
    }
    out[r] = pick;
  }
}

}  // namespace

RB_EXPORT int rb_sample(int* out, const float* logits, int64_t row_stride, int R, int V, const float* temperature,
                        const float* uniform, cudaStream_t stream) {
  if (R == 0) return 0;
  RB_REQUIRE(V > 0, "rb_sample: empty vocabulary");
  sample_kernel<<<R, THREADS, 0, stream>>>(out, logits, row_stride, V, temperature, uniform);
  RB_CHECK_LAUNCH("rb_sample");
  return 0;
}
