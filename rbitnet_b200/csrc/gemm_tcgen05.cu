// Tensor-core matrix product for sm_100a: C[tokens, out] = X[tokens, K] * W[out, K]^T, bfloat16
// operands, float32 accumulation in tensor memory.
//
// Orientation.  The weight matrix is the M side of the tcgen05 instruction (128 rows of W per
// CTA), the tokens are the N side (16..256 per CTA).  The same kernel therefore serves a
// prefill of thousands of tokens (N tile 256) and a decode step of 1..64 tokens (N tile 16..64)
// without wasting the 128-row M side on padding.  Both operands are K-major in shared memory:
// TMA brings [rows, 64] boxes of W and X with the 128-byte swizzle, which is the canonical
// K-major layout the instruction's shared-memory descriptors name.
//
// Roles in a CTA of 192 threads: warp 0 issues TMA loads into a ring of stages, warp 1 owns the
// tensor memory and issues tcgen05.mma (one lane), warps 2..5 read the accumulators back with
// tcgen05.ld and write the result.  With token tiles of at most 64 (which the caller asks for up
// to 256 tokens, where a product is bound by reading W) K may be cut into 2..8 parts: the CTAs
// of a tile then form a thread-block cluster, and after their products each of them adds up a
// share of the token columns from all parts, in part order, through distributed shared memory.
//
// Epilogues: plain store (bfloat16 or float32), add into a float32 matrix (the residual stream,
// crates/bitnet-core/src/llama/model.rs:291-294, :303-306),
// the q/k/v product of a decode step that rotates and appends to the cache (QkvTail below),
// and SiLU(gate)*up (model.rs:297-302) from ONE accumulator: the caller interleaves the rows of the
// gate and up matrices in blocks of 16, so that each warp of the epilogue holds 16 gate rows in its
// lower lanes and the 16 up rows of the same features in its upper lanes, and a shuffle pairs them.
//
// Every wait on an mbarrier is bounded: after about two seconds the waiting thread records an
// error code in a device word and the CTA leaves through the common exit, freeing its tensor
// memory.  The host reads the word with rb_read_error_flag().
#include "rb_tcgen05.cuh"

#include <mutex>
#include <unordered_map>
#include <string>

namespace {

constexpr int BM = 128;        // weight rows per CTA (UMMA M)
constexpr int BK = 64;         // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int W_TILE_BYTES = BM * BK * 2;

enum Epilogue { EPI_STORE = 0, EPI_ADD = 1, EPI_GATED = 3, EPI_QKV = 4 };     // (2 is not in use)

__host__ __device__ constexpr uint32_t make_idesc(int n) { return make_idesc_mn(BM, n, 0, 0); }

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

// What the q/k/v product of a few tokens does with its result instead of storing it (EPI_QKV):
// rotate the q and k heads by the token's position (crates/bitnet-core/src/llama/model.rs:122-136),
// write q to q_out [tokens, H, D], the rotated k and the raw v to the token's place in the paged
// cache (model.rs:254-257).  Rows of W: [H*D of q | Kh*D of k | Kh*D of v], or q alone.
struct QkvTail {
  __nv_bfloat16* q_out;
  const float* inv_freq;     // [D/2]
  const int* tok_pos;
  const int* tok_slot;
  RbPagedLayer cache;
  int H;
  int write_kv;              // 0: W holds q rows only (a layer that reads another layer's cache)
  int interleaved;           // pairs (2i, 2i+1) instead of (i, i + rot_dim/2)
  int rot_dim;               // the first rot_dim values of a head are rotated, the rest pass unchanged
};

struct GemmParams {
  void* C;            // output
  int64_t ldc;        // row stride of C in elements
  int n_tokens;       // rows of X
  int n_out;          // rows of W (for EPI_GATED: gate and up rows together)
  int K;
  int n_features;     // EPI_GATED: output columns (W holds 32 rows, 16 gate and 16 up, per 16 of them)
  int kb_per_split;   // 64-wide k blocks per split
  int n_t_tiles;      // token tiles
  int splits;         // parts of K
  int n_items;        // weight tiles * token tiles * splits
  int cluster;        // 1: the splits of a tile form a thread-block cluster and are summed through shared memory
  float alpha;        // multiplies the finished sum of a stored or added product (x * 1.0f is x exactly)
  QkvTail qkv;        // EPI_QKV only
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A CTA takes work items blockIdx.x, blockIdx.x + gridDim.x, ...; item = ((weight tile * token
// tiles) + token tile) * splits + split, so CTAs that run together share tiles of W and X in L2.
// When two accumulators fit in tensor memory they alternate, and the epilogue of one item runs
// while the tensor cores work on the next.
// MINB: CTAs that share an SM (2 for the small token tiles of a decode step: twice as many, smaller
// items stream W together and finish together, which evens out an item count that does not
// divide by the number of SMs).
template <int BN, int STAGES, int EPI, typename OutT, int MINB>
__global__ void __launch_bounds__(192, MINB)
gemm_wx_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GemmParams p) {
  constexpr int X_TILE_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
  constexpr int ACC_COLS = BN;
  constexpr int NBUF = 2 * ACC_COLS <= 512 ? 2 : 1;
  constexpr int WANT_COLS = NBUF * ACC_COLS;
  constexpr int TMEM_COLS = WANT_COLS <= 32 ? 32 : (WANT_COLS <= 64 ? 64 : (WANT_COLS <= 128 ? 128 : (WANT_COLS <= 256 ? 256 : 512)));
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
  static_assert(WANT_COLS <= 512, "tensor memory has 512 columns");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t accum_full[NBUF];
  __shared__ uint64_t accum_empty[NBUF];
  __shared__ uint32_t tmem_holder;

  rb_pdl_launch_dependents();     // the next kernel may be set up while this one runs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb_total = (p.K + BK - 1) / BK;
  // cluster mode: grid (splits, tiles), one item per CTA, blockIdx.x is the split and the cluster rank
  const int first_item = blockIdx.y * p.splits + blockIdx.x;
  const int item_stride = p.cluster ? p.n_items : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(&accum_full[b], 1);
      mbar_init(&accum_empty[b], 4);     // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_holder;
  // Barriers and tensor memory are ready.  Whoever touches memory that an earlier kernel may
  // still be writing or reading calls rb_pdl_wait() first: the loader before it loads X, the
  // epilogue warps before they touch C.  W is never written, so its first tiles are requested
  // before the wait and stream in while the kernel before this one finishes.

  // what an item covers
  auto item_of = [&](int item, int& n0, int& t0, int& kb_begin, int& nkb, int& split) {
    split = item % p.splits;
    const int tile = item / p.splits;
    n0 = (tile / p.n_t_tiles) * BM;
    t0 = (tile % p.n_t_tiles) * BN;
    kb_begin = split * p.kb_per_split;
    nkb = max(0, min(nkb_total, kb_begin + p.kb_per_split) - kb_begin);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      // the first item's first stages: W before the wait, X after it
      int early = 0;
      if (first_item < p.n_items) {
        int n0, t0, kb_begin, nkb, split;
        item_of(first_item, n0, t0, kb_begin, nkb, split);
        early = min(nkb, STAGES);
        for (int i = 0; i < early; ++i) {
          uint8_t* stage = smem + (size_t)i * STAGE_BYTES;
          mbar_expect_tx(&full_bar[i], STAGE_BYTES);
          const int k = (kb_begin + i) * BK;
          tma_load_2d(stage, &tmW, k, n0, &full_bar[i]);
        }
        rb_pdl_wait();
        for (int i = 0; i < early; ++i) {
          uint8_t* stage = smem + (size_t)i * STAGE_BYTES;
          tma_load_2d(stage + W_TILE_BYTES, &tmX, (kb_begin + i) * BK, t0, &full_bar[i]);
        }
      }
      for (int item = first_item; item < p.n_items && ok; item += item_stride) {
        int n0, t0, kb_begin, nkb, split;
        item_of(item, n0, t0, kb_begin, nkb, split);
        int i = 0;
        if (item == first_item) { i = early; it = early; }
        for (; i < nkb; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          ok = mbar_wait(&empty_bar[s], phase ^ 1, 1);
          if (!ok) break;
          uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          const int k = (kb_begin + i) * BK;
          tma_load_2d(stage, &tmW, k, n0, &full_bar[s]);
          tma_load_2d(stage + W_TILE_BYTES, &tmX, k, t0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      uint32_t it = 0, li = 0;
      bool ok = true;
      for (int item = first_item; item < p.n_items && ok; item += item_stride, ++li) {
        int n0, t0, kb_begin, nkb, split;
        item_of(item, n0, t0, kb_begin, nkb, split);
        const int b = li % NBUF;
        ok = mbar_wait(&accum_empty[b], ((li / NBUF) & 1) ^ 1, 4);    // the epilogue has drained this accumulator
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t acc_addr = tmem_base + (uint32_t)(b * ACC_COLS);
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          ok = mbar_wait(&full_bar[s], phase, 2);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t stage = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t dw = smem_desc_sw128(stage);
          const uint64_t dx = smem_desc_sw128(stage + W_TILE_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
            const uint32_t acc = (i > 0 || k4 > 0) ? 1u : 0u;
            const uint64_t koff = (uint64_t)(k4 * UMMA_K * 2 >> 4);
            umma_bf16(acc_addr, dw + koff, dx + koff, idesc, acc);
          }
          tcgen05_commit(&empty_bar[s]);   // frees the stage when these MMAs have read it
        }
        tcgen05_commit(&accum_full[b]);    // this item's accumulator is complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;        // tensor-memory lanes 32*quarter .. +31 belong to this warp
    rb_pdl_wait();                       // before C is read or written
    uint32_t li = 0;
    for (int item = first_item; item < p.n_items; item += item_stride, ++li) {
      int n0, t0, kb_begin, nkb, split;
      item_of(item, n0, t0, kb_begin, nkb, split);
      const int b = li % NBUF;
      const int n = n0 + quarter * 32 + lane;           // output column = weight row
      const bool n_ok = n < p.n_out;
      // EPI_ADD: the values to add to do not depend on the accumulator.  They are fetched one chunk
      // ahead, the first chunk while the products of this item still run, so that the epilogue
      // waits for memory once per item and not once per chunk.
      float ahead[16];
      auto fetch_old = [&](int c, float* into) {
        const int left = n_ok ? p.n_tokens - (t0 + c) : 0;
        const float* src = (const float*)p.C + (int64_t)(t0 + c) * p.ldc + n;
#pragma unroll
        for (int j = 0; j < 16; ++j) into[j] = j < left ? src[(int64_t)j * p.ldc] : 0.f;
      };
      if (EPI == EPI_ADD && !p.cluster) fetch_old(0, ahead);
      bool ok = true;
      if (lane == 0) ok = mbar_wait(&accum_full[b], (li / NBUF) & 1, 3);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tcgen05_fence_after();
      if (p.cluster) {
        // this split's accumulator goes to shared memory (the stage ring is idle now: every MMA
        // that read it has completed); the splits are added up after the cluster barrier below
        float* red = reinterpret_cast<float*>(smem);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (t0 + c >= p.n_tokens) break;
          uint32_t r[16];
          __syncwarp();
          if (nkb > 0) {
            tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * ACC_COLS + c), r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) red[(c + j) * BM + quarter * 32 + lane] = __uint_as_float(r[j]);
        }
        break;        // one item per CTA in this mode
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        if (t0 + c >= p.n_tokens) break;
        uint32_t r[16];
        __syncwarp();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * ACC_COLS + c);
        if (nkb > 0) {
          tmem_ld16(taddr, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
        // rows of this chunk that exist (none for a lane whose weight row is beyond the matrix);
        // no lane leaves the loop early: tcgen05.ld is executed by the whole warp
        const int t_left = n_ok ? p.n_tokens - (t0 + c) : 0;
        if (EPI == EPI_ADD) {
          float* dst = (float*)p.C + (int64_t)(t0 + c) * p.ldc + n;
          float old[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) old[j] = ahead[j];
          if (c + 16 < BN) fetch_old(c + 16, ahead);       // the next chunk's loads are in flight during these stores
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < t_left) dst[(int64_t)j * p.ldc] = old[j] + __uint_as_float(r[j]) * p.alpha;
        } else if (EPI == EPI_GATED) {
          // Lanes 0..15 hold gate rows, lanes 16..31 the up rows of the same 16 features (feature =
          // (weight row block of 32) * 16 + lane % 16).  Columns are taken in pairs: the lower lanes
          // finish the even token of a pair, the upper lanes the odd one, so that every lane does one
          // activation per two columns.  Every lane takes part in the shuffles.
          const bool low = lane < 16;
          const int f = (n0 + quarter * 32) / 2 + (lane & 15);
          const int f_left = f < p.n_features ? p.n_tokens - (t0 + c) : 0;
          OutT* dst = (OutT*)p.C + (int64_t)(t0 + c + (low ? 0 : 1)) * p.ldc + f;
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float mine = __uint_as_float(low ? r[j] : r[j + 1]);       // gate (low) or up (high) of my token
            const float send = __uint_as_float(low ? r[j + 1] : r[j]);       // what the partner needs
            const float got = __shfl_xor_sync(0xffffffffu, send, 16);
            const float g = low ? mine : got, up = low ? got : mine;
            // silu(g) * up = g * up / (1 + e^-g), with the hardware's exponential and reciprocal: their
            // error (a few units of float32) is far below the rounding to bfloat16 that follows
            const float v = __fdividef(g, 1.0f + __expf(-g)) * up;
            if (j + (low ? 0 : 1) < f_left) store_out<OutT>(dst + (int64_t)j * p.ldc, v);
          }
        } else {
          OutT* dst = (OutT*)p.C + (int64_t)(t0 + c) * p.ldc + n;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < t_left) store_out<OutT>(dst + (int64_t)j * p.ldc, __uint_as_float(r[j]) * p.alpha);
        }
      }
      // this warp has read its lanes of the accumulator: hand it back to the MMA issuer
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&accum_empty[b]);
    }
  }
  if (p.cluster) {
    // every thread of every CTA of the cluster arrives here, also after a wait that gave up
    static_assert(BN * BM * 4 <= STAGES * STAGE_BYTES, "the ring holds one accumulator");
    __syncwarp();
    cluster_sync_all();
    if (EPI == EPI_QKV && warp >= 2 && first_item < p.n_items) {
      // As below, every CTA of the cluster adds up its share of the token columns (column c belongs
      // to rank c mod splits).  The sums of this CTA's columns are then parked in its own shared
      // memory, behind the accumulators, so that a thread finds there the sum of the row its own row
      // is rotated with (both lie in this tile: the head size divides 128).  It rotates in float32
      // and writes the one rounded result where it belongs.  All four epilogue warps pass the
      // barrier between the two steps, whatever their rows.
      static_assert(BN > 64 || 2 * BN * BM * 4 <= STAGES * STAGE_BYTES, "the ring holds the accumulators and the sums");
      int n0, t0, kb_begin, nkb, split;
      item_of(first_item, n0, t0, kb_begin, nkb, split);
      const QkvTail& q = p.qkv;
      const int D = q.cache.head_dim, HD = q.H * D, KD = q.write_kv ? q.cache.n_kv_heads * D : 0;
      const int row = (warp & 3) * 32 + lane, n = n0 + row, d = n % D;
      const int my = (int)cluster_rank();
      const int R2 = q.rot_dim / 2;
      int pair = 0, prow = row;
      bool first = true;
      if (d < q.rot_dim) {
        if (q.interleaved) { pair = d >> 1; first = (d & 1) == 0; prow = row ^ 1; }
        else { pair = d % R2; first = d < R2; prow = first ? row + R2 : row - R2; }
      }
      const bool is_v = n >= HD + KD || d >= q.rot_dim, live = n < p.n_out;   // is_v: stored as it is
      float* sums = reinterpret_cast<float*>(smem) + BN * BM;       // [column][row], this CTA's columns only
      uint32_t own[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(own[r]) : "r"(smem_u32(smem) + (uint32_t)row * 4), "r"((uint32_t)(r < p.splits ? r : 0)));
      constexpr int CPI = BN >= 64 ? 4 : 2;                          // columns whose loads are in flight together
      if (live) {
        for (int cb = my; cb < BN && t0 + cb < p.n_tokens; cb += CPI * p.splits) {
          float part[CPI][8];
#pragma unroll
          for (int h = 0; h < CPI; ++h) {
            const int col = cb + h * p.splits;
            const bool ok = col < BN && t0 + col < p.n_tokens;
#pragma unroll
            for (int r = 0; r < 8; ++r) {      // all loads first, then the sums in split order
              part[h][r] = 0.f;
              if (ok && r < p.splits)
                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part[h][r]) : "r"(own[r] + (uint32_t)(col * BM) * 4));
            }
          }
#pragma unroll
          for (int h = 0; h < CPI; ++h) {
            const int col = cb + h * p.splits;
            if (col >= BN || t0 + col >= p.n_tokens) continue;
            float x = part[h][0];
#pragma unroll
            for (int r = 1; r < 8; ++r) x += part[h][r];
            sums[col * BM + row] = x;
          }
        }
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");                 // the four epilogue warps
      if (live) {
        const float inv = is_v ? 0.f : q.inv_freq[pair];
        for (int col = my; col < BN && t0 + col < p.n_tokens; col += p.splits) {
          const float x = sums[col * BM + row];
          const int t = t0 + col, pos = q.tok_pos[t];
          float y = x;
          if (!is_v) {
            const float xp = sums[col * BM + prow];
            float sn, cs;
            sincosf((float)pos * inv, &sn, &cs);
            y = first ? x * cs - xp * sn : xp * sn + x * cs;
          }
          __nv_bfloat16* dst;
          if (n < HD) dst = q.q_out + (int64_t)t * HD + n;
          else if (n < HD + KD) dst = (__nv_bfloat16*)q.cache.k + rb_page_offset(q.cache, q.tok_slot[t], pos, (n - HD) / D) + d;
          else dst = (__nv_bfloat16*)q.cache.v + rb_page_offset(q.cache, q.tok_slot[t], pos, (n - HD - KD) / D) + d;
          *dst = __float2bfloat16_rn(y);
        }
      }
    }
    if (EPI != EPI_GATED && EPI != EPI_QKV && warp >= 2 && first_item < p.n_items) {   // (the gated product is never split)
      // every CTA of the cluster adds up a share of the token columns (column c belongs to rank
      // c mod splits), reading all parts of a column in split order through distributed shared memory
      int n0, t0, kb_begin, nkb, split;
      item_of(first_item, n0, t0, kb_begin, nkb, split);
      const int quarter = warp & 3;
      const int n = n0 + quarter * 32 + lane;
      const int my = (int)cluster_rank();
      const uint32_t red = smem_u32(smem) + (uint32_t)(quarter * 32 + lane) * 4;
      uint32_t remote[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[r]) : "r"(red), "r"((uint32_t)(r < p.splits ? r : 0)));
      if (n < p.n_out) {
        constexpr int CPI = BN >= 64 ? 8 : (BN >= 32 ? 4 : 2);      // columns whose loads are in flight together
        for (int cb = 0; cb < BN; cb += CPI * p.splits) {
          int col[CPI];
          bool ok[CPI];
          float old[CPI], part[CPI][8];
#pragma unroll
          for (int h = 0; h < CPI; ++h) {
            col[h] = cb + h * p.splits + my;
            ok[h] = col[h] < BN && t0 + col[h] < p.n_tokens;
            old[h] = 0.f;
            if (EPI == EPI_ADD && ok[h]) old[h] = ((const float*)p.C)[(int64_t)(t0 + col[h]) * p.ldc + n];
          }
#pragma unroll
          for (int h = 0; h < CPI; ++h)
#pragma unroll
            for (int r = 0; r < 8; ++r) {      // all loads first, then the sums in split order
              part[h][r] = 0.f;
              if (ok[h] && r < p.splits)
                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part[h][r]) : "r"(remote[r] + (uint32_t)(col[h] * BM) * 4));
            }
#pragma unroll
          for (int h = 0; h < CPI; ++h) {
            if (!ok[h]) continue;
            float v = part[h][0];
#pragma unroll
            for (int r = 1; r < 8; ++r) v += part[h][r];
            v *= p.alpha;
            const int64_t at = (int64_t)(t0 + col[h]) * p.ldc + n;
            if (EPI == EPI_ADD) ((float*)p.C)[at] = old[h] + v;
            else store_out<OutT>((OutT*)p.C + at, v);
          }
        }
      }
    }
    __syncwarp();
    cluster_sync_all();        // nobody's shared memory goes away while another rank reads it
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct MapKey {
  const void* ptr; long long rows; int cols; int64_t ld; int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

// Tensor map of a row-major bfloat16 matrix [rows, cols] (cols contiguous), box [box_rows, 64],
// 128-byte swizzle, zero fill outside.  Maps are cached by their arguments: they are pure
// functions of them.
}  // namespace

int rb_get_tensor_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int64_t ld, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn fn = encode_fn();
  RB_REQUIRE(fn != nullptr, "rb_gemm: cuTensorMapEncodeTiled is not available from the driver");
  RB_REQUIRE(((uintptr_t)ptr & 15) == 0, "rb_gemm: matrix base %p is not 16-byte aligned", ptr);
  RB_REQUIRE((ld * 2) % 16 == 0, "rb_gemm: row stride of %lld elements is not a multiple of 8", (long long)ld);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RB_REQUIRE(r == CUDA_SUCCESS, "rb_gemm: cuTensorMapEncodeTiled failed with %d (rows %lld cols %d ld %lld)", (int)r,
             rows, cols, (long long)ld);
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return 0;
}

namespace {

template <int BN, int STAGES, int EPI, typename OutT, int MINB>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t stream) {
  constexpr int stage_bytes = W_TILE_BYTES + BN * BK * 2;
  constexpr int smem = STAGES * stage_bytes + 1024;
  static_assert(smem * MINB <= 227 * 1024, "shared memory");
  auto kernel = gemm_wx_kernel<BN, STAGES, EPI, OutT, MINB>;
  static RbOncePerDevice configured;
  if (configured.first()) {
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  }
  if (p.cluster) {
    // grid (splits, tiles): the CTAs of one tile are one cluster
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.splits, p.n_items / p.splits, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = rb_pdl_enabled() ? 2 : 1;
    RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, tw, tx, p));
    return 0;
  }
  const int slots = rb_sm_count() * MINB;
  const int grid = p.n_items < slots ? p.n_items : slots;     // resident CTAs take items in turn
  RB_LAUNCH("kernel", (kernel), grid, 192, smem, stream, tw, tx, p);
  RB_CHECK_LAUNCH("rb_gemm_tc");
  return 0;
}

template <int EPI, typename OutT>
int dispatch(int bn, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t stream) {
  switch (bn) {
    case 16: return launch<16, 5, EPI, OutT, 2>(tw, tx, p, stream);
    case 32: return launch<32, 5, EPI, OutT, 2>(tw, tx, p, stream);
    case 64: return launch<64, 4, EPI, OutT, 2>(tw, tx, p, stream);
    case 128: return launch<128, 6, EPI, OutT, 1>(tw, tx, p, stream);
    case 160: return launch<160, 5, EPI, OutT, 1>(tw, tx, p, stream);
    case 192: return launch<192, 5, EPI, OutT, 1>(tw, tx, p, stream);
    case 224: return launch<224, 4, EPI, OutT, 1>(tw, tx, p, stream);
    case 256: return launch<256, 4, EPI, OutT, 1>(tw, tx, p, stream);
  }
  RB_FAIL("rb_gemm_tc: no kernel for a token tile of %d", bn);
}

}  // namespace

// The device word that a kernel sets when one of its bounded waits ran out (0: none).
int rb_attention_tc_error_flag(int* value, int reset);   // attention_tcgen05.cu

int rb_attention_tc_error_flag_address(int** out);   // attention_tcgen05.cu

// Device addresses of the two error words, so that a step can report them with its results
// instead of the host reading them after every step.
RB_EXPORT int rb_error_flag_addresses(int** a, int** b) {
  if (rb_file_error_flag_address(a) != 0) return -1;
  return rb_attention_tc_error_flag_address(b);
}

RB_EXPORT int rb_read_error_flag(int* value, int reset) {
  int a = 0, b = 0;
  if (rb_file_error_flag(&a, reset) != 0) return -1;
  if (rb_attention_tc_error_flag(&b, reset) != 0) return -1;
  *value = a != 0 ? a : b;
  return 0;
}

// ---------------------------------------------------------------- the error word, for tests
// Writes `code` into the device error word, as a kernel whose wait ran out would: lets a test see
// the whole path from the word to the host's exception without any kernel waiting for anything.
RB_EXPORT int rb_set_error_flag_for_test(int code) { return rb_file_set_error_flag(code); }

// One thread waits on a barrier at which nobody ever arrives, with the given limit; the wait gives
// up, records `code` and the kernel returns.  This is the bounded wait of the product and attention
// kernels (same function, their limit is two seconds) run to its end on purpose, in a kernel that
// does nothing else.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int code, int* __restrict__ gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool ok = mbar_wait(&bar, 0, code, limit_ns);
    if (gave_up != nullptr) *gave_up = ok ? 0 : 1;
  }
}

RB_EXPORT int rb_wait_probe(long long limit_ns, int code, int* gave_up, cudaStream_t stream) {
  RB_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ll, "rb_wait_probe: limit %lld ns (at most 0.1 s)", limit_ns);
  wait_probe_kernel<<<1, 32, 0, stream>>>((unsigned long long)limit_ns, code, gave_up);
  RB_CHECK_LAUNCH("rb_wait_probe");
  return 0;
}

// Parts to cut the inner dimension of a product of n_tokens tokens into (the `splits` argument of
// rb_gemm_tc).  Up to 256 tokens a product is bound by reading W, so it wants every SM to stream a
// piece of it: the tokens go in tiles of at most 64, and when the 128-row tiles of W times the token
// tiles are fewer than the CTAs that run together (two per SM), K is cut as well: into 2, 4 or 8
// parts, the sizes clusters schedule well, each of at least four 64-wide blocks.  Beyond 256 tokens: one.
RB_EXPORT int rb_gemm_tc_splits(int n_tokens, int n_out, int K) {
  if (n_tokens > 256 || n_tokens <= 0 || n_out <= 0 || K <= 0) return 1;
  const int tiles = ((n_out + BM - 1) / BM) * ((n_tokens + 63) / 64);
  const int blocks = (K + BK - 1) / BK;
  const int together = 2 * rb_sm_count();
  int want = 1;
  while (want * 2 <= 8 && want * 2 <= together / tiles && want * 2 <= blocks / 4) want *= 2;
  const int per = (blocks + want - 1) / want;
  return (blocks + per - 1) / per;          // no part may be empty
}

// C (+)= X W^T on the tensor cores.
//   epilogue 0: C[tokens, n_out] = alpha * product, c_dtype float32 or bfloat16
//   epilogue 1: C (float32) += alpha * product
//   (epilogues 0 and 1 with 2..8 splits: the CTAs of a tile form a cluster and each adds up a share
//    of the token columns through distributed shared memory, in split order; token tile <= 64)
//   epilogue 3: W holds, for every 16 output features, 16 gate rows followed by their 16 up rows
//               (n_out rows in all, a multiple of 32); C[tokens, n_features] = silu(gate)*up
// Requirements (refused otherwise): bfloat16 X and W, K a multiple of 8, row strides multiples of 8
// elements, 16-byte aligned bases.
static int gemm_tc(void* C, int64_t ldc, int c_dtype, const void* X, int64_t ldx, int n_tokens, const void* W,
                   int64_t ldw, int w_rows, int n_out, int K, int epilogue, int n_features, int splits,
                   int token_tile, const QkvTail* tail, float alpha, cudaStream_t stream) {
  if (n_tokens == 0 || n_out == 0) return 0;
  RB_REQUIRE(alpha == 1.0f || epilogue == EPI_STORE || epilogue == EPI_ADD, "rb_gemm_tc: alpha %g with epilogue %d", alpha, epilogue);
  RB_REQUIRE(n_tokens > 0 && n_out > 0 && K > 0, "rb_gemm_tc: bad sizes tokens=%d out=%d K=%d", n_tokens, n_out, K);
  RB_REQUIRE(K % 8 == 0, "rb_gemm_tc: inner size %d is not a multiple of 8", K);
  RB_REQUIRE(splits >= 1, "rb_gemm_tc: splits %d", splits);
  RB_REQUIRE(epilogue != EPI_GATED || splits == 1, "rb_gemm_tc: the gated product cannot split K");
  RB_REQUIRE(splits <= 8, "rb_gemm_tc: at most 8 splits are summed on the device (%d asked)", splits);
  const int nkb = (K + BK - 1) / BK;
  RB_REQUIRE(splits <= nkb, "rb_gemm_tc: %d splits for %d blocks of K", splits, nkb);
  int bn = token_tile;
  if (bn == 0) {
    bn = n_tokens <= 16 ? 16 : n_tokens <= 32 ? 32 : n_tokens <= 64 ? 64 : n_tokens <= 128 ? 128 : 256;
    if (n_tokens > 128 && n_tokens <= 4096) {
      // Few enough tokens that tiles of 256 may leave most SMs without an item, or with a last round
      // of few: take the tile (128 to 256 tokens in steps of 32) that needs the least time, counted as
      // rounds of the SMs times what an item costs.  An item of 128 tokens costs about 0.7 of one
      // of 256, not half (measured: with half, a 1,024-token prefill took 16.7 ms instead of 13.9
      // because the gate/up product moved to 128); between them the cost is taken as linear.  Measured
      // against tiles of 128 and 256 alone: 300 tokens 7.6 ms instead of 8.2, 768 tokens 10.5 instead
      // of 11.35, 1,200 tokens 16.7 instead of 18.2, 1,500 tokens 19.2 instead of 20.4; 2,048 and 4,096
      // tokens take 256 as before.  Beyond 4,096 tokens the rounds are many and 256 stays.
      const long long w_tiles = (n_out + BM - 1) / BM, sms = rb_sm_count();
      double best = 0.0;
      for (int cand = 128; cand <= 256; cand += 32) {
        const long long rounds = (w_tiles * ((n_tokens + cand - 1) / cand) + sms - 1) / sms;
        const double cost = (double)rounds * (0.4 + 0.6 * cand / 256.0);
        if (cand == 128 || cost < best - 1e-9) { best = cost; bn = cand; }
      }
    }
  }
  RB_REQUIRE(epilogue != EPI_GATED || (n_out % 32 == 0 && n_features > 0 && n_features <= n_out / 2),
             "rb_gemm_tc: the gated product wants rows in blocks of 32 (%d rows, %d features)", n_out, n_features);
  CUtensorMap tw, tx;
  if (rb_get_tensor_map(&tw, W, w_rows, K, ldw, BM) != 0) return -1;
  if (rb_get_tensor_map(&tx, X, n_tokens, K, ldx, bn) != 0) return -1;
  GemmParams p;
  p.C = C; p.ldc = ldc; p.n_tokens = n_tokens; p.n_out = n_out; p.K = K;
  p.n_features = n_features; p.kb_per_split = (nkb + splits - 1) / splits;
  RB_REQUIRE((int64_t)(splits - 1) * p.kb_per_split < nkb, "rb_gemm_tc: a split of K would be empty");
  const int n_w_tiles = (n_out + BM - 1) / BM, n_t_tiles = (n_tokens + bn - 1) / bn;
  const long long items = (long long)n_w_tiles * n_t_tiles * splits;
  RB_REQUIRE(items < (1ll << 30), "rb_gemm_tc: too many tiles");
  p.n_t_tiles = n_t_tiles; p.splits = splits; p.n_items = (int)items;
  p.cluster = splits > 1 ? 1 : 0;
  p.alpha = alpha;
  RB_REQUIRE(!p.cluster || bn <= 64, "rb_gemm_tc: K is split only for token tiles of at most 64");
  if (epilogue == EPI_QKV) {
    RB_REQUIRE(tail != nullptr && p.cluster, "rb_gemm_tc: the q/k/v tail wants K split into a cluster");
    p.qkv = *tail;
    return dispatch<EPI_QKV, __nv_bfloat16>(bn, tw, tx, p, stream);
  }
  if (epilogue == EPI_STORE && c_dtype == RB_BF16) return dispatch<EPI_STORE, __nv_bfloat16>(bn, tw, tx, p, stream);
  if (epilogue == EPI_STORE && c_dtype == RB_F32) return dispatch<EPI_STORE, float>(bn, tw, tx, p, stream);
  if (epilogue == EPI_ADD && c_dtype == RB_F32) return dispatch<EPI_ADD, float>(bn, tw, tx, p, stream);
  if (epilogue == EPI_GATED && c_dtype == RB_BF16) return dispatch<EPI_GATED, __nv_bfloat16>(bn, tw, tx, p, stream);
  RB_FAIL("rb_gemm_tc: unsupported epilogue %d with output dtype %d", epilogue, c_dtype);
}

RB_EXPORT int rb_gemm_tc(void* C, int64_t ldc, int c_dtype, const void* X, int64_t ldx, int n_tokens, const void* W,
                         int64_t ldw, int w_rows, int n_out, int K, int epilogue, int n_features, int splits,
                         int token_tile, float alpha, cudaStream_t stream) {
  RB_REQUIRE(epilogue == EPI_STORE || epilogue == EPI_ADD || epilogue == EPI_GATED, "rb_gemm_tc: unknown epilogue %d", epilogue);
  return gemm_tc(C, ldc, c_dtype, X, ldx, n_tokens, W, ldw, w_rows, n_out, K, epilogue, n_features, splits, token_tile,
                 nullptr, alpha, stream);
}

// Whether rb_gemm_tc_qkv takes these sizes: a head may not straddle two 128-row tiles of W, and the
// product must be one that is split along K (2..8 parts).  At most 16 tokens: with 64, the rotation
// in the epilogue (also with the sines and cosines made once per step) measured slower than the
// rotation kernel it saves (9,490 against 9,840 tokens/s).
RB_EXPORT int rb_gemm_tc_qkv_supports(int n_tokens, int D, int splits) {
  return n_tokens >= 1 && n_tokens <= 16 && splits >= 2 && splits <= 8 && D >= 2 && D % 2 == 0 && BM % D == 0;
}

// The q/k/v product of up to 16 tokens with rotation and cache append in its epilogue (see QkvTail).
// W: [H*D + (write_kv ? 2*Kh*D : 0), K].  K is cut into `splits` >= 2 parts (one cluster per tile).
RB_EXPORT int rb_gemm_tc_qkv(void* q_out, const void* X, int64_t ldx, int n_tokens, const void* W, int64_t ldw, int K,
                             int splits, const float* inv_freq, const int* tok_pos, const int* tok_slot, void* cache_k,
                             void* cache_v, const int* page_table, int max_pages, int page_size, int H, int Kh, int D,
                             int write_kv, int interleaved, int rot_dim, cudaStream_t stream) {
  RB_REQUIRE(rb_gemm_tc_qkv_supports(n_tokens, D, splits), "rb_gemm_tc_qkv: tokens=%d head=%d splits=%d not supported",
             n_tokens, D, splits);
  RB_REQUIRE(H > 0 && Kh >= 0 && page_size > 0, "rb_gemm_tc_qkv: bad sizes H=%d Kh=%d page=%d", H, Kh, page_size);
  RB_REQUIRE(rot_dim >= 0 && rot_dim <= D && rot_dim % 2 == 0,
             "rb_gemm_tc_qkv: the rotated prefix %d must be even and at most the head size %d", rot_dim, D);
  QkvTail tail;
  tail.q_out = (__nv_bfloat16*)q_out; tail.inv_freq = inv_freq; tail.tok_pos = tok_pos; tail.tok_slot = tok_slot;
  tail.cache = RbPagedLayer{cache_k, cache_v, page_table, max_pages, page_size, Kh, D};
  tail.H = H; tail.write_kv = write_kv ? 1 : 0; tail.interleaved = interleaved ? 1 : 0;
  tail.rot_dim = rot_dim;
  const int rows = (H + (write_kv ? 2 * Kh : 0)) * D;
  return gemm_tc(q_out, (int64_t)H * D, RB_BF16, X, ldx, n_tokens, W, ldw, rows, rows, K, EPI_QKV, 0, splits, 0, &tail,
                 1.0f, stream);
}

RB_CHECK_READER(gemm_tcgen05)
