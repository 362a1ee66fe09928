// Next-token choice on the device.
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
//
// Two launches.  Pass 1 cuts each row into chunks (grid rows x chunks): per chunk the
// max, the lowest index holding it, and the sum of exp((z - chunk max)/T).  Pass 2
// (one block per row) merges the chunks, finds the chunk the target falls into, and
// walks that chunk with a block-wide running sum in index order.  `stats` is scratch
// of rows * chunks * 3 floats.
#include "rb_common.cuh"

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ float clean(float v) { return v != v ? -INFINITY : v; }

__global__ void __launch_bounds__(THREADS) sample_stats_kernel(float* __restrict__ stats,
                                                              const float* __restrict__ logits, int64_t row_stride,
                                                              int V, int chunk, const float* __restrict__ temperature) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  __shared__ float scratch[33];
  __shared__ int s_arg;
  const int r = blockIdx.x, c = blockIdx.y, n_chunks = gridDim.y;
  const float* z = logits + (int64_t)r * row_stride;
  const int lo = min(V, c * chunk), hi = min(V, lo + chunk);
  float m = -INFINITY;
  for (int i = lo + threadIdx.x; i < hi; i += THREADS) m = fmaxf(m, clean(z[i]));
  m = rb_block_max(m, scratch);
  if (threadIdx.x == 0) s_arg = V;
  __syncthreads();
  int best = V;
  for (int i = lo + threadIdx.x; i < hi; i += THREADS)
    if (clean(z[i]) == m) { best = i; break; }
  if (best < V) atomicMin(&s_arg, best);
  const float temp = temperature[r];
  float sum = 0.f;
  if (temp > 0.f && m > -INFINITY) {
    const float inv_t = 1.0f / temp;
    for (int i = lo + threadIdx.x; i < hi; i += THREADS) sum += expf((clean(z[i]) - m) * inv_t);
  }
  sum = rb_block_sum(sum, scratch);
  if (threadIdx.x == 0) {
    float* o = stats + ((int64_t)r * n_chunks + c) * 3;
    o[0] = m;
    o[1] = __int_as_float(s_arg);
    o[2] = sum;
  }
}

__global__ void __launch_bounds__(THREADS) sample_pick_kernel(int* __restrict__ out, const float* __restrict__ stats,
                                                             const float* __restrict__ logits, int64_t row_stride,
                                                             int V, int chunk, int n_chunks,
                                                             const float* __restrict__ temperature,
                                                             const float* __restrict__ uniform) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  __shared__ float part[THREADS];
  __shared__ float s_m, s_before, s_target;
  __shared__ int s_chunk, s_pick;
  const int r = blockIdx.x;
  const float* st = stats + (int64_t)r * n_chunks * 3;
  const float* z = logits + (int64_t)r * row_stride;
  const float temp = temperature[r];
  if (threadIdx.x == 0) {
    float m = -INFINITY;
    int arg = V;
    for (int c = 0; c < n_chunks; ++c) {
      const float mc = st[c * 3];
      const int ac = __float_as_int(st[c * 3 + 1]);
      if (mc > m) { m = mc; arg = ac; }          // chunks ascend, so the first max holds the lowest index
    }
    s_m = m;
    s_chunk = -1;
    s_pick = arg < V ? arg : 0;
    if (temp > 0.f && m > -INFINITY) {
      const float inv_t = 1.0f / temp;
      float total = 0.f;
      for (int c = 0; c < n_chunks; ++c) total += st[c * 3 + 2] * expf((st[c * 3] - m) * inv_t);
      const float target = uniform[r] * total;
      float before = 0.f;
      int pick = n_chunks - 1;
      for (int c = 0; c < n_chunks; ++c) {
        const float sc = st[c * 3 + 2] * expf((st[c * 3] - m) * inv_t);
        if (before + sc >= target) { pick = c; break; }
        if (c < n_chunks - 1) before += sc;
      }
      s_chunk = pick;
      s_before = before;
      s_target = target;
      s_pick = V - 1;                            // if rounding leaves the target past the end
    }
  }
  __syncthreads();
  if (s_chunk < 0) {
    if (threadIdx.x == 0) out[r] = s_pick;
    return;
  }
  // walk the chosen chunk (and what follows, if rounding pushed the target past it) in index order
  const float inv_t = 1.0f / temp, m = s_m;
  float before = s_before;
  const float target = s_target;
  for (int lo = s_chunk * chunk; lo < V; lo += chunk) {
    const int hi = min(V, lo + chunk);
    const int per = (hi - lo + THREADS - 1) / THREADS;
    const int a = min(hi, lo + threadIdx.x * per), b = min(hi, a + per);
    float local = 0.f;
    for (int i = a; i < b; ++i) local += expf((clean(z[i]) - m) * inv_t);
    part[threadIdx.x] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
      float c = before;
      int owner = -1;
      for (int t = 0; t < THREADS; ++t) {
        if (c + part[t] >= target) { owner = t; break; }
        c += part[t];
      }
      s_chunk = owner;           // reused: the thread whose elements hold the target, or -1
      s_before = c;              // running sum before that thread's elements (or after the whole chunk)
    }
    __syncthreads();
    if (s_chunk >= 0) {
      if (threadIdx.x == s_chunk) {
        float c = s_before;
        int pick = b - 1;
        for (int i = a; i < b; ++i) {
          c += expf((clean(z[i]) - m) * inv_t);
          if (c >= target) { pick = i; break; }
        }
        out[r] = pick;
      }
      return;
    }
    before = s_before;
    __syncthreads();
  }
  if (threadIdx.x == 0) out[r] = V - 1;
}

}  // namespace

RB_EXPORT int rb_sample_chunks(int V) {
  const int c = (V + 4095) / 4096;
  return c < 1 ? 1 : (c > 64 ? 64 : c);
}

// stats: rows * rb_sample_chunks(V) * 3 floats of scratch.
RB_EXPORT int rb_sample(int* out, const float* logits, int64_t row_stride, int R, int V, const float* temperature,
                        const float* uniform, float* stats, cudaStream_t stream) {
  if (R == 0) return 0;
  RB_REQUIRE(V > 0, "rb_sample: empty vocabulary");
  RB_REQUIRE(stats != nullptr, "rb_sample: no scratch");
  const int n_chunks = rb_sample_chunks(V);
  const int chunk = (V + n_chunks - 1) / n_chunks;
  RB_LAUNCH("sample_stats_kernel", (sample_stats_kernel), dim3(R, n_chunks), THREADS, 0, stream, stats, logits, row_stride, V, chunk, temperature);
  RB_CHECK_LAUNCH("rb_sample (stats)");
  RB_LAUNCH("sample_pick_kernel", (sample_pick_kernel), R, THREADS, 0, stream, out, stats, logits, row_stride, V, chunk, n_chunks, temperature, uniform);
  RB_CHECK_LAUNCH("rb_sample (pick)");
  return 0;
}
