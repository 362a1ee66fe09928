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
// Token tiles of 128 and more leave through shared memory as TMA boxes (an added product is added by
// the memory system), and an added product of many tokens may share its weight tiles between teams
// of CTAs; for up to 16 tokens the RMS norm between two products (model.rs:93-100) rides in their
// epilogues.  The kernel's own comment has each of these.
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

// The kernel's third tensor map, that of the output, exists only where the output leaves by TMA:
// elsewhere the parameter is one word.
template <bool BY_TMA> struct OutputMap { using type = CUtensorMap; };
template <> struct OutputMap<false> { struct type { int none; }; };
template <int BN, int EPI> constexpr bool leaves_by_tma() { return BN >= 128 && EPI != EPI_QKV; }

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
  // Shared ranges (sk_len > 0; token tiles of 128 and more, no cluster): see the kernel's comment.
  int sk_len;         // 64-wide k blocks per team of CTAs
  int n_w_tiles;      // 128-row tiles of W
  int* sk_finished;   // [weight tile][token tile]: parts of the tile that are in C; zero between launches
  // A norm that whoever made X left pending (norm_ss != nullptr; token tiles of 16): X holds
  // the rows times the norm's weights, and the finished sums of token t are multiplied by
  // 1 / sqrt(sum over parts of norm_ss[part][t] / norm_width + norm_eps).
  const float* norm_ss;
  int norm_parts;
  float norm_width, norm_eps;
  // EPI_ADD in a cluster, for the norm that follows: also leaves bfloat16(C_new * emit_g[column]) in
  // emit_xb [tokens, emit_ld] and the sums of squares of C_new over every warp's 32 columns in
  // emit_ss [4 * weight tiles][tokens].
  __nv_bfloat16* emit_xb;
  int64_t emit_ld;
  const float* emit_g;
  float* emit_ss;
  QkvTail qkv;        // EPI_QKV only
};

// What one pass of a CTA's three roles covers: k blocks kb_begin .. kb_begin + nkb - 1 of the tile
// at (n0, t0).  With shared ranges a tile's K may be covered by `parts` teams, of which this is
// number `part` (teams first_team .. first_team + parts - 1, in the order of their k blocks).
struct Piece {
  int n0, t0, kb_begin, nkb;
  int w_tile, part, parts, first_team;
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
//
// Shared ranges (p.sk_len > 0; products added to C, token tiles of 128 and more).  Tiles in turn
// leave SMs idle in the last round whenever the tiles are not a multiple of the SMs (2,048 tokens
// times 4,096 rows: 256 tiles on 148 SMs take two rounds for 1.73 rounds of work).  Here the CTAs
// form teams of as many CTAs as there are token tiles; the k blocks of all weight tiles, laid end to
// end, are cut into equal ranges, one per team, and the CTAs of a team walk the team's range
// together, each on its own token tile, so that a tile of W is still fetched once for all token
// tiles.  Where a range begins or ends inside a weight tile, that tile's K is shared by two or more
// teams.  Each adds its part to C (the memory system does the addition, as for a whole tile), and
// the parts are added in the order of their k blocks, so that the sum is the same every time: a
// part's first box waits until the tile's count of finished parts has reached the part's number.  A
// part that waits is never the first piece of a range that ends inside a tile, which is the piece
// that holds the tile's first k blocks and is taken first; so the part that everybody else waits
// for waits for nobody, all CTAs of the launch are resident (one per SM at most), and every wait is
// bounded like the others.  The last part sets the count back to zero.
template <int BN, int STAGES, int EPI, typename OutT, int MINB>
__global__ void __launch_bounds__(192, MINB)
gemm_wx_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
               const __grid_constant__ typename OutputMap<leaves_by_tma<BN, EPI>()>::type tmC, GemmParams p) {
  constexpr int X_TILE_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
  constexpr int ACC_COLS = BN;
  constexpr int NBUF = 2 * ACC_COLS <= 512 ? 2 : 1;
  constexpr int WANT_COLS = NBUF * ACC_COLS;
  constexpr int TMEM_COLS = WANT_COLS <= 32 ? 32 : (WANT_COLS <= 64 ? 64 : (WANT_COLS <= 128 ? 128 : (WANT_COLS <= 256 ? 256 : 512)));
  constexpr bool SHARED_RANGES = BN >= 128 && EPI == EPI_ADD;     // compiled in for these only
  // Token tiles of 128 and more leave through shared memory: 16 token rows of the tile at a time are
  // staged there and go out as one TMA box (stored, or added to the residual stream by the memory
  // system), two boxes in flight.  Stores a thread makes itself have one chunk of loads or stores in
  // flight per thread, about 8 KB an SM, and an epilogue of a 128 x 256 tile then takes longer than
  // the products of a short tile.
  constexpr bool TMA_EPI = leaves_by_tma<BN, EPI>();
  // A pending norm of the input rows and what a later norm needs (see GemmParams) are compiled for the
  // 16-token tile only, which is where a step uses them: present in the 64-token tile's kernels, asked
  // for or not, they cost each product of a batch of 64 about half a microsecond.
  constexpr bool PENDING_NORM = BN <= 16;
  constexpr int OUT_COLS = EPI == EPI_GATED ? BM / 2 : BM;          // values per token row of a staged box
  constexpr int OUT_STAGE_BYTES = 16 * BM * 4;                      // room for 16 rows of float32
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
  static_assert(WANT_COLS <= 512, "tensor memory has 512 columns");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* out_stage = smem + (size_t)STAGES * STAGE_BYTES;          // TMA_EPI: two boxes of OUT_STAGE_BYTES
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t accum_full[NBUF];
  __shared__ uint64_t accum_empty[NBUF];
  __shared__ uint32_t tmem_holder;
  __shared__ int epi_fail;
  __shared__ float norm_r[64];         // per token: the factor of a pending norm

  rb_pdl_launch_dependents();     // the next kernel may be set up while this one runs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb_total = (p.K + BK - 1) / BK;
  // cluster mode: grid (splits, tiles), one item per CTA, blockIdx.x is the split and the cluster rank
  const int first_item = blockIdx.y * p.splits + blockIdx.x;
  const int item_stride = p.cluster ? p.n_items : gridDim.x;

  if (threadIdx.x == 0) {
    epi_fail = 0;
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

  // the li-th piece of this CTA's work (false: there is none)
  const bool shared_ranges = SHARED_RANGES && p.sk_len > 0;
  const int sk_team = shared_ranges ? (int)blockIdx.x / p.n_t_tiles : 0;
  const int sk_tt = shared_ranges ? (int)blockIdx.x % p.n_t_tiles : 0;
  auto piece_at = [&](int li, Piece& s) -> bool {
    if (SHARED_RANGES && shared_ranges) {
      const long long begin = (long long)sk_team * p.sk_len;
      const long long total = (long long)p.n_w_tiles * nkb_total;
      const long long end = begin + p.sk_len < total ? begin + p.sk_len : total;
      // Pieces in the order of their k blocks: g0, g0 + 1, ..., g_last.  A piece that ends the range
      // inside a weight tile is taken first instead of last: then both shared pieces of a team come
      // before its whole tiles, whose products hide the passing of the parts through memory.
      const int g0 = (int)(begin / nkb_total), g_last = (int)((end - 1) / nkb_total);
      if (begin >= end || li > g_last - g0) return false;
      const bool last_first = g_last > g0 && end < (long long)(g_last + 1) * nkb_total;
      const int g = last_first ? (li == 0 ? g_last : g0 + li - 1) : g0 + li;
      const long long from = g == g0 ? begin : (long long)g * nkb_total;
      const long long g_begin = (long long)g * nkb_total, g_end = g_begin + nkb_total;
      const long long to = g_end < end ? g_end : end;
      s.w_tile = g;
      s.n0 = g * BM;
      s.t0 = sk_tt * BN;
      s.kb_begin = (int)(from - g_begin);
      s.nkb = (int)(to - from);
      s.first_team = (int)(g_begin / p.sk_len);
      s.parts = (int)((g_end - 1) / p.sk_len) - s.first_team + 1;
      s.part = sk_team - s.first_team;
      return true;
    }
    const int item = first_item + li * item_stride;
    if (item >= p.n_items) return false;
    const int split = item % p.splits;
    const int tile = item / p.splits;
    s.w_tile = tile / p.n_t_tiles;
    s.n0 = s.w_tile * BM;
    s.t0 = (tile % p.n_t_tiles) * BN;
    s.kb_begin = split * p.kb_per_split;
    s.nkb = max(0, min(nkb_total, s.kb_begin + p.kb_per_split) - s.kb_begin);
    s.part = 0; s.parts = 1; s.first_team = 0;
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      // the first piece's first stages: W before the wait, X after it
      int early = 0;
      Piece s;
      if (piece_at(0, s)) {
        early = min(s.nkb, STAGES);
        for (int i = 0; i < early; ++i) {
          uint8_t* stage = smem + (size_t)i * STAGE_BYTES;
          mbar_expect_tx(&full_bar[i], STAGE_BYTES);
          const int k = (s.kb_begin + i) * BK;
          tma_load_2d(stage, &tmW, k, s.n0, &full_bar[i]);
        }
        rb_pdl_wait();
        for (int i = 0; i < early; ++i) {
          uint8_t* stage = smem + (size_t)i * STAGE_BYTES;
          tma_load_2d(stage + W_TILE_BYTES, &tmX, (s.kb_begin + i) * BK, s.t0, &full_bar[i]);
        }
      }
      for (int li = 0; ok && piece_at(li, s); ++li) {
        int i = 0;
        if (li == 0) { i = early; it = early; }
        for (; i < s.nkb; ++i, ++it) {
          const int st = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          ok = mbar_wait(&empty_bar[st], phase ^ 1, 1);
          if (!ok) break;
          uint8_t* stage = smem + (size_t)st * STAGE_BYTES;
          mbar_expect_tx(&full_bar[st], STAGE_BYTES);
          const int k = (s.kb_begin + i) * BK;
          tma_load_2d(stage, &tmW, k, s.n0, &full_bar[st]);
          tma_load_2d(stage + W_TILE_BYTES, &tmX, k, s.t0, &full_bar[st]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      uint32_t it = 0;
      bool ok = true;
      Piece s;
      for (int li = 0; ok && piece_at(li, s); ++li) {
        const int nkb = s.nkb;
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
    const int row = quarter * 32 + lane;
    const bool issuer = warp == 2 && lane == 0;      // the one thread that sends the boxes of TMA_EPI
    rb_pdl_wait();                       // before C is read or written
    const bool normed = PENDING_NORM && p.norm_ss != nullptr;
    if (normed) {
      // (the parts are summed in their order, by one thread per token: the same sum in every CTA)
      const int t = (int)threadIdx.x - 64;
      if (t < 64) {
        float r = 1.0f;
        if (t < p.n_tokens) {
          float ss = 0.f;
          for (int q = 0; q < p.norm_parts; ++q) ss += p.norm_ss[(int64_t)q * p.n_tokens + t];
          r = 1.0f / sqrtf(ss / p.norm_width + p.norm_eps);
        }
        norm_r[t] = r;
      }
      asm volatile("bar.sync 3, 128;" ::: "memory");
    }
    uint32_t n_boxes = 0;
    Piece s;
    for (int li = 0; piece_at(li, s); ++li) {
      const int n0 = s.n0, t0 = s.t0, nkb = s.nkb;
      const int b = li % NBUF;
      const int n = n0 + row;                           // output column = weight row
      const bool n_ok = n < p.n_out;
      // EPI_ADD without TMA: the values to add to do not depend on the accumulator.  They are fetched
      // one chunk ahead, the first chunk while the products of this item still run, so that the
      // epilogue waits for memory once per item and not once per chunk.
      float ahead[16];
      auto fetch_old = [&](int c, float* into) {
        const int left = n_ok ? p.n_tokens - (t0 + c) : 0;
        const float* src = (const float*)p.C + (int64_t)(t0 + c) * p.ldc + n;
#pragma unroll
        for (int j = 0; j < 16; ++j) into[j] = j < left ? src[(int64_t)j * p.ldc] : 0.f;
      };
      if (EPI == EPI_ADD && !TMA_EPI && !p.cluster) fetch_old(0, ahead);
      bool ok = true;
      if (lane == 0) ok = mbar_wait(&accum_full[b], (li / NBUF) & 1, 3);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (TMA_EPI) {
        // the four warps meet at barriers below: they go on together or leave together
        if (!ok && lane == 0) epi_fail = 1;
        asm volatile("bar.sync 3, 128;" ::: "memory");
        ok = *(volatile int*)&epi_fail == 0;
      }
      if (!ok) break;
      tcgen05_fence_after();
      // columns c .. c+15 of this warp's 32 rows of the accumulator
      auto load_acc = [&](int c, uint32_t (&r)[16]) {
        __syncwarp();
        if (nkb > 0) {
          tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * ACC_COLS + c), r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
      };
      if (p.cluster) {
        // this split's accumulator goes to shared memory (the stage ring is idle now: every MMA
        // that read it has completed); the splits are added up after the cluster barrier below
        float* red = reinterpret_cast<float*>(smem);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (t0 + c >= p.n_tokens) break;
          uint32_t r[16];
          load_acc(c, r);
#pragma unroll
          for (int j = 0; j < 16; ++j) red[(c + j) * BM + row] = __uint_as_float(r[j]);
        }
        break;        // one item per CTA in this mode
      }
      if constexpr (TMA_EPI) {
        // A tile whose K is shared: the parts are added to C in the order of their k blocks, so this
        // part's first box waits until the count of finished parts has reached its own number.
        int* finished = nullptr;
        bool must_wait = false;
        if (SHARED_RANGES && s.parts > 1) {
          finished = p.sk_finished + (int64_t)s.w_tile * p.n_t_tiles + sk_tt;
          must_wait = s.part > 0;
        }
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (t0 + c >= p.n_tokens) break;
          uint32_t r[16];
          load_acc(c, r);
          // The 16 token rows of the chunk go to shared memory as [token][OUT_COLS values] and leave as
          // one box; rows and columns beyond the matrix are dropped by the tensor map.
          OutT* box = reinterpret_cast<OutT*>(out_stage + (n_boxes & 1) * OUT_STAGE_BYTES);
          ++n_boxes;
          if (EPI == EPI_GATED) {
            // Lanes 0..15 hold gate rows, lanes 16..31 the up rows of the same 16 features (feature =
            // (weight row block of 32) * 16 + lane % 16).  Columns are taken in pairs: the lower lanes
            // finish the even token of a pair, the upper lanes the odd one, so that every lane does one
            // activation per two columns.  Every lane takes part in the shuffles.
            const bool low = lane < 16;
            OutT* dst = box + (low ? 0 : OUT_COLS) + quarter * 16 + (lane & 15);
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              const float mine = __uint_as_float(low ? r[j] : r[j + 1]);       // gate (low) or up (high) of my token
              const float send = __uint_as_float(low ? r[j + 1] : r[j]);       // what the partner needs
              const float got = __shfl_xor_sync(0xffffffffu, send, 16);
              const float g = low ? mine : got, up = low ? got : mine;
              // silu(g) * up = g * up / (1 + e^-g), with the hardware's exponential and reciprocal: their
              // error (a few units of float32) is far below the rounding to bfloat16 that follows
              store_out<OutT>(dst + j * OUT_COLS, __fdividef(g, 1.0f + __expf(-g)) * up);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) store_out<OutT>(box + j * OUT_COLS + row, __uint_as_float(r[j]) * p.alpha);
          }
          fence_async_shared();
          if (issuer) bulk_wait_read_all();          // the box before this one has left its half of the staging area
          asm volatile("bar.sync 3, 128;" ::: "memory");
          if (issuer) {
            if (must_wait) {
              if (!wait_for_count(finished, s.part, 4)) epi_fail = 1;     // noticed at the next piece; the results are void
              must_wait = false;
            }
            tma_store_2d(&tmC, box, EPI == EPI_GATED ? n0 / 2 : n0, t0 + c, EPI == EPI_ADD);
            bulk_commit();
          }
        }
        if (finished != nullptr && issuer) {
          // this part is in C: count it, or, as the last part, set the count back for the next launch
          bulk_wait_all();
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          const int now = s.part + 1 == s.parts ? 0 : s.part + 1;
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(finished), "r"(now) : "memory");
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (t0 + c >= p.n_tokens) break;
          uint32_t r[16];
          load_acc(c, r);
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
              if (j < t_left)
                dst[(int64_t)j * p.ldc] = old[j] + __uint_as_float(r[j]) * (normed ? p.alpha * norm_r[t0 + c + j] : p.alpha);
          } else if (EPI == EPI_GATED) {
            // as above, each lane storing its own values
            const bool low = lane < 16;
            const int f = (n0 + quarter * 32) / 2 + (lane & 15);
            const int f_left = f < p.n_features ? p.n_tokens - (t0 + c) : 0;
            OutT* dst = (OutT*)p.C + (int64_t)(t0 + c + (low ? 0 : 1)) * p.ldc + f;
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              const float mine = __uint_as_float(low ? r[j] : r[j + 1]);
              const float send = __uint_as_float(low ? r[j + 1] : r[j]);
              const float got = __shfl_xor_sync(0xffffffffu, send, 16);
              const float rr = normed ? norm_r[t0 + c + j + (low ? 0 : 1)] : 1.0f;       // my token's pending norm
              const float g = (low ? mine : got) * rr, up = (low ? got : mine) * rr;
              const float v = __fdividef(g, 1.0f + __expf(-g)) * up;
              if (j + (low ? 0 : 1) < f_left) store_out<OutT>(dst + (int64_t)j * p.ldc, v);
            }
          } else {
            OutT* dst = (OutT*)p.C + (int64_t)(t0 + c) * p.ldc + n;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < t_left)
                store_out<OutT>(dst + (int64_t)j * p.ldc, __uint_as_float(r[j]) * (normed ? p.alpha * norm_r[t0 + c + j] : p.alpha));
          }
        }
      }
      // this warp has read its lanes of the accumulator: hand it back to the MMA issuer
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&accum_empty[b]);
    }
    if (TMA_EPI && issuer) bulk_wait_all();      // the last boxes are in global memory
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
      Piece pc;
      piece_at(0, pc);
      const int n0 = pc.n0, t0 = pc.t0;
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
        const bool normed = PENDING_NORM && p.norm_ss != nullptr;
        for (int col = my; col < BN && t0 + col < p.n_tokens; col += p.splits) {
          const int t = t0 + col, pos = q.tok_pos[t];
          const float rr = normed ? norm_r[t] : 1.0f;            // a pending norm of the input rows
          const float x = sums[col * BM + row] * rr;
          float y = x;
          if (!is_v) {
            const float xp = sums[col * BM + prow] * rr;
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
    if (EPI != EPI_QKV && warp >= 2 && first_item < p.n_items) {
      // every CTA of the cluster adds up a share of the token columns (column c belongs to rank
      // c mod splits), reading all parts of a column in split order through distributed shared memory
      Piece pc;
      piece_at(0, pc);
      const int n0 = pc.n0, t0 = pc.t0;
      const int quarter = warp & 3;
      const int n = n0 + quarter * 32 + lane;
      const int my = (int)cluster_rank();
      const uint32_t red = smem_u32(smem) + (uint32_t)(quarter * 32 + lane) * 4;
      uint32_t remote[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[r]) : "r"(red), "r"((uint32_t)(r < p.splits ? r : 0)));
      // (every lane walks the loop, also one whose weight row is beyond the matrix: the warp adds up
      // squares together below)
      const bool n_in = n < p.n_out;
      const bool normed = PENDING_NORM && p.norm_ss != nullptr;
      constexpr bool CAN_EMIT = EPI == EPI_ADD && PENDING_NORM;
      const bool emit = CAN_EMIT && p.emit_xb != nullptr;
      const float g_n = emit && n_in ? p.emit_g[n] : 0.f;
      {
        constexpr int CPI = BN >= 64 ? 8 : (BN >= 32 ? 4 : 2);      // columns whose loads are in flight together
        for (int cb = 0; cb < BN; cb += CPI * p.splits) {
          int col[CPI];
          bool ok[CPI];
          float old[CPI], part[CPI][8];
#pragma unroll
          for (int h = 0; h < CPI; ++h) {
            col[h] = cb + h * p.splits + my;
            ok[h] = n_in && col[h] < BN && t0 + col[h] < p.n_tokens;
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
            const bool column = col[h] < BN && t0 + col[h] < p.n_tokens;       // the same in every lane
            if (EPI == EPI_GATED) {
              // lanes 0..15 hold the gate sums of 16 features, lanes 16..31 their up sums (see the epilogue
              // above): every lane adds up its parts, the halves meet by a shuffle, the lower lanes finish
              float v = part[h][0];
#pragma unroll
              for (int r = 1; r < 8; ++r) v += part[h][r];
              if (normed) v *= norm_r[column ? t0 + col[h] : 0];
              const float up = __shfl_xor_sync(0xffffffffu, v, 16);
              const int f = (n0 + quarter * 32) / 2 + (lane & 15);
              if (ok[h] && lane < 16 && f < p.n_features)
                store_out<OutT>((OutT*)p.C + (int64_t)(t0 + col[h]) * p.ldc + f, __fdividef(v, 1.0f + __expf(-v)) * up);
              continue;
            }
            float now = 0.f;
            if (ok[h]) {
              float v = part[h][0];
#pragma unroll
              for (int r = 1; r < 8; ++r) v += part[h][r];
              v *= normed ? p.alpha * norm_r[t0 + col[h]] : p.alpha;
              const int64_t at = (int64_t)(t0 + col[h]) * p.ldc + n;
              if (EPI == EPI_ADD) {
                now = old[h] + v;
                ((float*)p.C)[at] = now;
                if (emit) p.emit_xb[(int64_t)(t0 + col[h]) * p.emit_ld + n] = __float2bfloat16_rn(now * g_n);
              } else {
                store_out<OutT>((OutT*)p.C + at, v);
              }
            }
            if (emit && column) {
              // the squares of this warp's 32 columns of C, lane 0 .. lane 31 in a fixed tree
              float sq = now * now;
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
              if (lane == 0) p.emit_ss[(int64_t)((n0 / BM) * 4 + quarter) * p.n_tokens + t0 + col[h]] = sq;
            }
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
  int box_cols, elem_bytes;        // 0, 0: a bfloat16 operand (box of 64 columns, 128-byte swizzle)
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && elem_bytes == o.elem_bytes;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    h = h * 1000003u ^ (size_t)k.box_rows;
    h = h * 1000003u ^ (size_t)(k.box_cols * 8 + k.elem_bytes);
    return h;
  }
};

// Tensor map of a row-major bfloat16 matrix [rows, cols] (cols contiguous), box [box_rows, 64],
// 128-byte swizzle, zero fill outside.  Maps are cached by their arguments: they are pure
// functions of them.
}  // namespace

static int get_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int64_t ld, int box_rows, int box_cols,
                   int elem_bytes) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows, box_cols, elem_bytes};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  const bool operand = elem_bytes == 0;
  const int eb = operand ? 2 : elem_bytes;
  EncodeTiledFn fn = encode_fn();
  RB_REQUIRE(fn != nullptr, "rb_gemm: cuTensorMapEncodeTiled is not available from the driver");
  RB_REQUIRE(((uintptr_t)ptr & 15) == 0, "rb_gemm: matrix base %p is not 16-byte aligned", ptr);
  RB_REQUIRE((ld * eb) % 16 == 0, "rb_gemm: row stride of %lld elements is not a multiple of %d", (long long)ld, 16 / eb);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * eb};
  cuuint32_t box[2] = {(cuuint32_t)(operand ? BK : box_cols), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, operand || eb == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  operand ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  operand ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RB_REQUIRE(r == CUDA_SUCCESS, "rb_gemm: cuTensorMapEncodeTiled failed with %d (rows %lld cols %d ld %lld)", (int)r,
             rows, cols, (long long)ld);
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return 0;
}

int rb_get_tensor_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int64_t ld, int box_rows) {
  return get_map(out, ptr, rows, cols, ld, box_rows, 0, 0);
}

int rb_get_output_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int64_t ld, int box_rows, int box_cols,
                      int elem_bytes) {
  RB_REQUIRE(elem_bytes == 2 || elem_bytes == 4, "rb_get_output_map: element of %d bytes", elem_bytes);
  return get_map(out, ptr, rows, cols, ld, box_rows, box_cols, elem_bytes);
}

namespace {

thread_local int t_kernels_launched = 0;     // by this thread's product calls, for tests

template <int BN, int STAGES, int EPI, typename OutT, int MINB>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tc, const GemmParams& p, cudaStream_t stream) {
  constexpr int stage_bytes = W_TILE_BYTES + BN * BK * 2;
  constexpr int smem = STAGES * stage_bytes + 1024 + (BN >= 128 ? 2 * 16 * BM * 4 : 0);
  static_assert(smem * MINB <= 227 * 1024, "shared memory");
  auto kernel = gemm_wx_kernel<BN, STAGES, EPI, OutT, MINB>;
  ++t_kernels_launched;
  typename OutputMap<leaves_by_tma<BN, EPI>()>::type out_map;
  if constexpr (leaves_by_tma<BN, EPI>()) out_map = tc; else out_map.none = 0;
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
    RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, tw, tx, out_map, p));
    return 0;
  }
  const int slots = rb_sm_count() * MINB;
  int grid = p.n_items < slots ? p.n_items : slots;     // resident CTAs take items in turn
  if (p.sk_len > 0) {
    RB_REQUIRE(BN >= 128 && EPI == EPI_ADD && p.n_items <= slots, "rb_gemm_tc: shared ranges with a token tile of %d, %d CTAs", BN, p.n_items);
    grid = p.n_items;                                    // one CTA per team and token tile
  }
  RB_LAUNCH("kernel", (kernel), grid, 192, smem, stream, tw, tx, out_map, p);
  RB_CHECK_LAUNCH("rb_gemm_tc");
  return 0;
}

template <int EPI, typename OutT>
int dispatch(int bn, const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tc, const GemmParams& p,
             cudaStream_t stream) {
  switch (bn) {
    case 16: return launch<16, 5, EPI, OutT, 2>(tw, tx, tc, p, stream);
    case 32: return launch<32, 5, EPI, OutT, 2>(tw, tx, tc, p, stream);
    case 64: return launch<64, 4, EPI, OutT, 2>(tw, tx, tc, p, stream);
    case 128: return launch<128, 6, EPI, OutT, 1>(tw, tx, tc, p, stream);
    case 160: return launch<160, 5, EPI, OutT, 1>(tw, tx, tc, p, stream);
    case 192: return launch<192, 5, EPI, OutT, 1>(tw, tx, tc, p, stream);
    case 224: return launch<224, 4, EPI, OutT, 1>(tw, tx, tc, p, stream);
    case 256: return launch<256, 4, EPI, OutT, 1>(tw, tx, tc, p, stream);
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

// The same for the wait on a count in global memory (a tile's finished parts): `word` holds zero and
// nobody ever stores the one that the thread waits for.
__global__ void count_wait_probe_kernel(const int* __restrict__ word, unsigned long long limit_ns, int code,
                                        int* __restrict__ gave_up) {
  if (threadIdx.x == 0) {
    const bool ok = wait_for_count(word, 1, code, limit_ns);
    if (gave_up != nullptr) *gave_up = ok ? 0 : 1;
  }
}

RB_EXPORT int rb_count_wait_probe(const int* word, long long limit_ns, int code, int* gave_up, cudaStream_t stream) {
  RB_REQUIRE(word != nullptr && limit_ns > 0 && limit_ns <= 100000000ll, "rb_count_wait_probe: limit %lld ns (at most 0.1 s)", limit_ns);
  count_wait_probe_kernel<<<1, 32, 0, stream>>>(word, (unsigned long long)limit_ns, code, gave_up);
  RB_CHECK_LAUNCH("rb_count_wait_probe");
  return 0;
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

// ---------------------------------------------------------------- shared ranges: the plan and the counters
namespace {
constexpr int SK_MAX_COUNTS = 1 << 16;             // tiles whose finished parts can be counted
struct SkWorkspace { void* ptr = nullptr; long long bytes = 0; };
SkWorkspace g_sk_ws[64];
std::mutex g_sk_mu;
int g_sk_len_for_test = 0;       // > 0: k blocks per team whatever the estimate says (tests)
int g_tail_for_test = 0;         // < 0: a last round of few tiles stays in the one product (tests, measurements)

double item_cost(int bn) { return 0.4 + 0.6 * bn / 256.0; }

struct GemmPlan { int bn; int sk_len; int teams; int n_t; double cost; };

// Tiles in turn against shared ranges for one token tile: the estimated time in units of one item of
// 256 tokens.  In turn: rounds of the SMs.  Shared ranges (`shared_ok`: an added product with
// counters to use): the weight tiles divided among the teams (SMs / token tiles of them); and since
// the parts of a shared tile are added to C one after the other, as many times the leaving of a tile
// as the tile with the most parts has parts.  A tile of 256 tokens that is added to C takes about as
// long to leave as 12 of its k blocks take to multiply (5 us against 0.4 us; measured on 4,096 rows
// times 4,096 and 14,336 with 300, 1,200 and 2,048 tokens).
GemmPlan plan_for_tile(int n_tokens, int n_out, int K, int bn, int sms, bool shared_ok) {
  const long long w_tiles = (n_out + BM - 1) / BM, n_t = (n_tokens + bn - 1) / bn, nkb = (K + BK - 1) / BK;
  GemmPlan pl{bn, 0, 0, (int)n_t, 0.0};
  const long long rounds = (w_tiles * n_t + sms - 1) / sms;
  pl.cost = (double)rounds * item_cost(bn);
  if (!shared_ok || bn < 128 || n_t > sms || w_tiles * n_t > SK_MAX_COUNTS) return pl;
  const double leaving = 12.0 / nkb * bn / 256.0;
  pl.cost += leaving;
  const long long teams = sms / n_t, total = w_tiles * nkb;
  long long len = (total + teams - 1) / teams;
  len = (len + 3) / 4 * 4;                       // no part shorter than four k blocks where K allows it
  const bool forced = g_sk_len_for_test > 0 && g_sk_len_for_test >= (total + teams - 1) / teams;
  if (forced) len = g_sk_len_for_test;
  if (len >= (1ll << 30)) return pl;
  const long long used = (total + len - 1) / len;
  const long long most_parts = len >= nkb ? 2 : (nkb + len - 1) / len + 1;
  const double shared_cost = (double)len / nkb * item_cost(bn) + most_parts * leaving;
  if (forced || shared_cost < pl.cost - 1e-9) { pl.cost = forced ? 0.0 : shared_cost; pl.sk_len = (int)len; pl.teams = (int)used; }
  return pl;
}

GemmPlan plan_gemm(int n_tokens, int n_out, int K, int token_tile, int sms, bool shared_ok) {
  if (token_tile != 0) return plan_for_tile(n_tokens, n_out, K, token_tile, sms, shared_ok);
  const int bn = n_tokens <= 16 ? 16 : n_tokens <= 32 ? 32 : n_tokens <= 64 ? 64 : n_tokens <= 128 ? 128 : 256;
  GemmPlan best = plan_for_tile(n_tokens, n_out, K, bn, sms, shared_ok);
  if (n_tokens > 128) {
    // Take the token tile (128 to 256 in steps of 32) that needs the least time.  An item of 128
    // tokens costs about 0.7 of one of 256, not half (measured: with half, a 1,024-token prefill
    // took 16.7 ms instead of 13.9 because the gate/up product moved to 128); between them the cost
    // is taken as linear.
    for (int cand = 128; cand <= 256; cand += 32) {
      const GemmPlan pl = plan_for_tile(n_tokens, n_out, K, cand, sms, shared_ok);
      if (cand == 128 || pl.cost < best.cost - 1e-9) best = pl;
    }
  }
  return best;
}
}  // namespace

// Bytes of device memory that rb_gemm_tc_set_workspace wants.
RB_EXPORT long long rb_gemm_tc_workspace_bytes() { return (long long)SK_MAX_COUNTS * 4; }

// Gives the products of the current device their counters for shared ranges (see the kernel): they
// must be zero, and the kernels leave them zero.  Products on different streams must not overlap in
// time: they share them.  Without them (or with ptr == nullptr, which takes them away) tiles are
// taken in turn.
RB_EXPORT int rb_gemm_tc_set_workspace(void* ptr, long long bytes) {
  int dev = 0;
  RB_CUDA(cudaGetDevice(&dev));
  RB_REQUIRE(dev >= 0 && dev < 64, "rb_gemm_tc_set_workspace: device %d", dev);
  RB_REQUIRE(ptr == nullptr || (bytes >= (long long)SK_MAX_COUNTS * 4 && ((uintptr_t)ptr & 15) == 0),
             "rb_gemm_tc_set_workspace: %lld bytes at %p, wanted %lld, 16-byte aligned", bytes, ptr, (long long)SK_MAX_COUNTS * 4);
  std::lock_guard<std::mutex> g(g_sk_mu);
  g_sk_ws[dev].ptr = ptr;
  g_sk_ws[dev].bytes = ptr ? bytes : 0;
  return 0;
}

// For tests: added products share their weight tiles with this many k blocks per team (if the SMs
// suffice for that), whatever the estimate says; 0 takes it back.
RB_EXPORT int rb_gemm_tc_share_for_test(int blocks_per_team) {
  RB_REQUIRE(blocks_per_team >= 0, "rb_gemm_tc_share_for_test: %d", blocks_per_team);
  g_sk_len_for_test = blocks_per_team;
  return 0;
}

// Kernels that this thread's rb_gemm_tc and rb_gemm_tc_qkv calls have launched so far (a product may be two).
RB_EXPORT int rb_gemm_tc_kernels_launched() { return t_kernels_launched; }

// For tests and measurements: -1 keeps a last round of few tiles in the one product; 0 takes it back.
RB_EXPORT int rb_gemm_tc_tail_for_test(int mode) {
  g_tail_for_test = mode;
  return 0;
}

// What rb_gemm_tc would do with these sizes on a device of `sms` SMs: out = {token tile, k blocks
// per team (0: tiles in turn), teams, token tiles}.  `shared_ok`: an added product (epilogue 1) on a
// device that has its counters.  No device is touched.
RB_EXPORT int rb_gemm_tc_plan(int n_tokens, int n_out, int K, int token_tile, int sms, int shared_ok, int* out) {
  RB_REQUIRE(n_tokens > 0 && n_out > 0 && K > 0 && sms > 0 && out != nullptr, "rb_gemm_tc_plan: bad arguments");
  const GemmPlan pl = plan_gemm(n_tokens, n_out, K, token_tile, sms, shared_ok != 0);
  out[0] = pl.bn; out[1] = pl.sk_len; out[2] = pl.teams; out[3] = pl.n_t;
  return 0;
}

// ---------------------------------------------------------------- a norm between two products
// The product that adds to the residual stream can leave what the norm after it needs, and the
// product after the norm can finish it, so that a decode step has no kernel for the norm: see
// GemmParams.  Both requests hold for the NEXT rb_gemm_tc or rb_gemm_tc_qkv call of the calling
// thread and are forgotten after it, whether it succeeded or not.
namespace {
struct NormOptions {
  const float* in_ss = nullptr; int in_parts = 0; float in_width = 0.f, in_eps = 0.f;
  void* out_xb = nullptr; int64_t out_ld = 0; const float* out_g = nullptr; float* out_ss = nullptr;
};
thread_local NormOptions t_norm;
}  // namespace

// The rows of X are rows * norm weight with the norm's factor pending: ss [parts, n_tokens] float32
// holds sums of squares of the rows (over `width` values in all).  At most 16 tokens.
RB_EXPORT int rb_gemm_tc_pending_norm(const float* ss, int parts, float width, float eps) {
  RB_REQUIRE(ss != nullptr && parts > 0 && width > 0.f, "rb_gemm_tc_pending_norm: bad arguments");
  t_norm.in_ss = ss; t_norm.in_parts = parts; t_norm.in_width = width; t_norm.in_eps = eps;
  return 0;
}

// The next product (epilogue 1, at most 16 tokens, K split into a cluster) also leaves bfloat16(C_new * g[column]) in
// xb [n_tokens, ld] and sums of squares of C_new in ss [rb_gemm_tc_norm_parts(n_out), n_tokens].
RB_EXPORT int rb_gemm_tc_leave_norm(void* xb, int64_t ld, const float* g, float* ss) {
  RB_REQUIRE(xb != nullptr && g != nullptr && ss != nullptr && ld > 0, "rb_gemm_tc_leave_norm: bad arguments");
  t_norm.out_xb = xb; t_norm.out_ld = ld; t_norm.out_g = g; t_norm.out_ss = ss;
  return 0;
}

// Rows of the sums of squares that rb_gemm_tc_leave_norm fills for n_out output columns.
RB_EXPORT int rb_gemm_tc_norm_parts(int n_out) { return 4 * ((n_out + BM - 1) / BM); }

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
  const NormOptions norm = t_norm;
  t_norm = NormOptions();
  if (n_tokens == 0 || n_out == 0) return 0;
  RB_REQUIRE(alpha == 1.0f || epilogue == EPI_STORE || epilogue == EPI_ADD, "rb_gemm_tc: alpha %g with epilogue %d", alpha, epilogue);
  RB_REQUIRE(n_tokens > 0 && n_out > 0 && K > 0, "rb_gemm_tc: bad sizes tokens=%d out=%d K=%d", n_tokens, n_out, K);
  RB_REQUIRE(K % 8 == 0, "rb_gemm_tc: inner size %d is not a multiple of 8", K);
  RB_REQUIRE(splits >= 1, "rb_gemm_tc: splits %d", splits);
  RB_REQUIRE(splits <= 8, "rb_gemm_tc: at most 8 splits are summed on the device (%d asked)", splits);
  const int nkb = (K + BK - 1) / BK;
  RB_REQUIRE(splits <= nkb, "rb_gemm_tc: %d splits for %d blocks of K", splits, nkb);
  SkWorkspace ws;
  if (splits == 1 && epilogue == EPI_ADD) {
    int dev = 0;
    RB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> g(g_sk_mu);
    if (dev >= 0 && dev < 64) ws = g_sk_ws[dev];
  }
  GemmPlan plan = plan_gemm(n_tokens, n_out, K, token_tile, rb_sm_count(), ws.ptr != nullptr);
  // token tiles of 128 and more write their output by TMA, which wants a 16-byte aligned base and row
  // stride; an output that is not (a width of 257 bfloat16 values) takes tiles of 64, which store by themselves
  const int out_elem = (epilogue == EPI_ADD || c_dtype == RB_F32) ? 4 : 2;
  if (plan.bn >= 128 && (((uintptr_t)C & 15) != 0 || (ldc * out_elem) % 16 != 0))
    plan = plan_for_tile(n_tokens, n_out, K, 64, rb_sm_count(), false);
  const int bn = plan.bn;
  RB_REQUIRE(epilogue != EPI_GATED || (n_out % 32 == 0 && n_features > 0 && n_features <= n_out / 2),
             "rb_gemm_tc: the gated product wants rows in blocks of 32 (%d rows, %d features)", n_out, n_features);
  // A last round of few tiles.  Tiles in turn pay a whole round of the SMs for it (2,048 tokens times
  // 28,672 rows: 1,792 tiles are twelve rounds of 148 SMs and 16 tiles, whatever power of two times
  // 224 the tiles are).  The weight tiles that whole rounds hold stay one product; the few that are
  // left become a second one on all SMs: token tiles of 64, K cut into a cluster, as for few tokens.
  if (token_tile == 0 && bn >= 128 && splits == 1 && plan.sk_len == 0 && g_tail_for_test >= 0 &&
      (epilogue == EPI_GATED || epilogue == EPI_STORE)) {
    const long long sms = rb_sm_count(), w_tiles = (n_out + BM - 1) / BM, n_t = (n_tokens + bn - 1) / bn;
    const long long items = w_tiles * n_t, rounds = (items + sms - 1) / sms, left = items - (rounds - 1) * sms;
    const long long w_main = (rounds - 1) * sms / n_t, w_tail = w_tiles - w_main;
    const long long tail_tiles = w_tail * ((n_tokens + 63) / 64);
    int parts = 1;
    while (parts * 2 <= 8 && tail_tiles * parts * 2 <= 2 * sms && parts * 2 <= nkb / 4) parts *= 2;
    // What the second product costs against the round it replaces, in microseconds.  Its tiles of 64 tokens
    // are bound by what they fetch, every token tile its own copy of the rows of W (128 + 64 rows of K
    // values a tile, at about 5 TB/s from L2), plus its start and its cluster's sum; a round is an item's k
    // blocks at 0.4 us each for 256 tokens.  Measured at 4,096 values of K and 28,672 rows: 300 tokens 87 us
    // instead of 99, 512 106 instead of 117, 1,024 171 instead of 180, 1,500 241 instead of 242; at 2,048 and
    // 4,096 tokens the second product would be the longer one (314 against 311, 620 against 598).
    const double tail_us = (double)tail_tiles * (BM + 64) * K * 2 / 5e6 + 4.0;
    const double round_us = nkb * 0.4 * item_cost(bn);
    if (rounds >= 2 && left * 4 <= sms && w_main >= 1 && w_tail >= 1 && parts >= 2 && tail_us < 0.8 * round_us) {
      const int rows_main = (int)w_main * BM;
      const int64_t out_off = epilogue == EPI_GATED ? rows_main / 2 : rows_main;       // columns of C the main product fills
      const int feat_main = epilogue == EPI_GATED ? (n_features < out_off ? n_features : (int)out_off) : 0;
      if (gemm_tc(C, ldc, c_dtype, X, ldx, n_tokens, W, ldw, rows_main, rows_main, K, epilogue, feat_main, 1, bn, nullptr,
                  alpha, stream) != 0)
        return -1;
      if (epilogue == EPI_GATED && n_features <= out_off) return 0;                      // the rest is padding rows
      char* c_tail = (char*)C + out_off * out_elem;
      const char* w_rest = (const char*)W + (int64_t)rows_main * ldw * 2;
      const int per = (nkb + parts - 1) / parts;
      return gemm_tc(c_tail, ldc, c_dtype, X, ldx, n_tokens, w_rest, ldw, w_rows - rows_main, n_out - rows_main, K, epilogue,
                     epilogue == EPI_GATED ? n_features - (int)out_off : 0, (nkb + per - 1) / per, 64, nullptr, alpha, stream);
    }
  }
  CUtensorMap tw, tx;
  if (rb_get_tensor_map(&tw, W, w_rows, K, ldw, BM) != 0) return -1;
  if (rb_get_tensor_map(&tx, X, n_tokens, K, ldx, bn) != 0) return -1;
  CUtensorMap tc = tw;               // token tiles below 128 store by themselves
  if (bn >= 128 && epilogue != EPI_QKV) {
    const int cols = epilogue == EPI_GATED ? n_features : n_out;
    if (rb_get_output_map(&tc, C, n_tokens, cols, ldc, 16, epilogue == EPI_GATED ? BM / 2 : BM, out_elem) != 0) return -1;
  }
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
  p.norm_ss = norm.in_ss; p.norm_parts = norm.in_parts; p.norm_width = norm.in_width; p.norm_eps = norm.in_eps;
  RB_REQUIRE(norm.in_ss == nullptr || (bn <= 16 && n_tokens <= 16),
             "rb_gemm_tc: a pending norm with %d tokens in tiles of %d (at most 16 tokens)", n_tokens, bn);
  p.emit_xb = (__nv_bfloat16*)norm.out_xb; p.emit_ld = norm.out_ld; p.emit_g = norm.out_g; p.emit_ss = norm.out_ss;
  RB_REQUIRE(norm.out_xb == nullptr || (epilogue == EPI_ADD && p.cluster && bn <= 16),
             "rb_gemm_tc: only an added product of at most 16 tokens whose K is split into a cluster leaves a norm's inputs");
  p.n_w_tiles = n_w_tiles;
  p.sk_len = plan.sk_len;
  p.sk_finished = (int*)ws.ptr;
  if (p.sk_len > 0) {
    p.n_items = plan.teams * n_t_tiles;        // CTAs: one per team and token tile
  }
  RB_REQUIRE(!p.cluster || bn <= 64, "rb_gemm_tc: K is split only for token tiles of at most 64");
  if (epilogue == EPI_QKV) {
    RB_REQUIRE(tail != nullptr && p.cluster, "rb_gemm_tc: the q/k/v tail wants K split into a cluster");
    p.qkv = *tail;
    return dispatch<EPI_QKV, __nv_bfloat16>(bn, tw, tx, tc, p, stream);
  }
  if (epilogue == EPI_STORE && c_dtype == RB_BF16) return dispatch<EPI_STORE, __nv_bfloat16>(bn, tw, tx, tc, p, stream);
  if (epilogue == EPI_STORE && c_dtype == RB_F32) return dispatch<EPI_STORE, float>(bn, tw, tx, tc, p, stream);
  if (epilogue == EPI_ADD && c_dtype == RB_F32) return dispatch<EPI_ADD, float>(bn, tw, tx, tc, p, stream);
  if (epilogue == EPI_GATED && c_dtype == RB_BF16) return dispatch<EPI_GATED, __nv_bfloat16>(bn, tw, tx, tc, p, stream);
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
