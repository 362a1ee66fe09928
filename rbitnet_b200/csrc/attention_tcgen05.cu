// Prefill attention on the 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05.mma
// with the accumulators in tensor memory; keys and values come from the paged cache by TMA.
//
// One CTA works for ONE kv head of ONE sequence on a tile of 128 rows; a row is a (token, query
// head) pair of the heads that share the kv head (row r -> token r / G, head kvh*G + r % G), so
// the G heads of a group reuse every key and value tile.  Keys and values arrive in tiles of 128
// positions (two 64-position pieces, each one page or an aligned part of a page), two stages each.
// The instructions are as wide as the head allows (N = 128 keys for S, N = D for O): narrow
// tcgen05.mma run far below the tensor cores' rate.
//
// Roles (320 threads): warp 0 loads K and V tiles with TMA; warp 1 owns tensor memory and issues
// the MMAs; warps 2..9 are the softmax, two threads per row (64 keys each).  Per key tile:
//   MMA:      S[128, 128] = Q[128, D] K[128, D]^T                   (bfloat16 in, float32 in TMEM)
//   softmax:  read the row of S, mask by position (causal, window), running max and sum in
//             float32, rescale the row of O in tensor memory when the max grew much, round P to
//             bfloat16 into tensor memory, in place of S (the A operand of the next MMA)
//   MMA:      O[128, D] += P[128, 128] V[128, D]
// S has two buffers: S of the next tile is issued before P V of this one, so the tensor cores work
// while the softmax runs.  The score is (q.k)*scale with the scale folded into the exponent (base 2).
// crates/bitnet-core/src/llama/model.rs:260-289 (scores, mask by loop bound, P V), :102-114 (softmax).
//
// The A operands of both products live in tensor memory: Q is written there once (two bfloat16 per
// column), and P overwrites the S it was made from.  The products therefore read only K and V from
// shared memory, which is what bounds N = 128 products whose operands both come from there.  K is
// K-major with the 128-byte swizzle; V, whose tile [keys, D] has D contiguous, is the MN-major B
// operand of O += P V.  Every mbarrier wait is bounded.
#include "rb_tcgen05.cuh"

namespace {

constexpr int ROWS = 128;          // rows of a CTA (UMMA M)
constexpr int TILE_KEYS = 128;     // keys per tile (UMMA N of S, K of P V)
constexpr int PIECE = 64;          // positions per TMA piece of a tile (a page, or an aligned part of one)
constexpr int THREADS = 320;       // loader warp, MMA warp, eight softmax warps
constexpr int KV_STAGES = 2;

struct TcAttnParams {
  const __nv_bfloat16* q;   // [T, H, D]
  __nv_bfloat16* out;       // [T, H*D]
  const int* page_table;
  int max_pages, page_size, n_kv_heads;
  const int* tok_pos;
  const int* tok_slot;
  const int* tile_tok0;
  const int* tile_ntok;
  int n_tiles;
  int H, G;
  float scale_log2;
  int window;
};

// 2^x for x <= 0 (and -inf -> 0) with the hardware approximation (relative error about 2^-22)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed float32 pairs (one instruction for two values) and the three-input maximum of sm_100.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// MN-major operand (the contiguous dimension is M or N), 128-byte swizzle: 64 contiguous elements
// per row of 128 bytes, eight K rows per group of 1024 bytes; `lbo` is the distance between
// 64-element blocks along M/N.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t saddr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows, 16 bfloat16 = 8 columns of 32 bits per
// row) is read from tensor memory instead of shared memory.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int D>
struct TcSmem {
  static constexpr int DB = D / 64;                         // 64-column blocks of a head
  static constexpr int BLOCK = ROWS * 128;                  // a block of [128 rows][128 bytes]
  static constexpr int KV_TILE_BYTES = BLOCK * DB;          // 128 keys, DB blocks
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_TILE_BYTES;
  static constexpr int OFF_MAX = OFF_V + KV_STAGES * KV_TILE_BYTES;   // float [2 tiles][2 halves][128 rows]
  static constexpr int OFF_BAR = OFF_MAX + 2 * 2 * ROWS * 4;
  static constexpr int BYTES = OFF_BAR + 128;
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, TcAttnParams p) {
  using S = TcSmem<D>;
  constexpr int DB = S::DB;
  // tensor memory: two S buffers in columns [0,256), O in [256, 256+D), Q (two bfloat16 a column) after it
  constexpr int O_COL = 2 * TILE_KEYS;
  constexpr int Q_COL = O_COL + D;
  constexpr int TMEM_COLS = 512;
  static_assert(2 * TILE_KEYS + D + D / 2 <= 512, "tensor memory columns");
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* k_full = bars;                   // [2] keys of a tile have landed
  uint64_t* k_empty = bars + 2;              // [2] S of that tile is complete: the key stage is free
  uint64_t* v_full = bars + 4;               // [2]
  uint64_t* v_empty = bars + 6;              // [2] P V of that tile is complete
  uint64_t* s_full = bars + 8;               // [2] one per S buffer
  uint64_t* p_full = bars + 10;              // P of a tile is in tensor memory (one arrival per softmax warp)
  uint64_t* pv_done = bars + 11;             // P V of a tile is complete: O is consistent, the P buffer is free
  uint64_t* o_full = bars + 12;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 13);
  float* row_max = reinterpret_cast<float*>(smem + S::OFF_MAX);

  rb_pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // late tiles see the most keys: CTAs start in the order (tile descending, kv head), so the long
  // ones of every kv head run first and the short ones fill the end
  const int tile = p.n_tiles - 1 - (int)blockIdx.y;
  const int kvh = blockIdx.x;
  const int G = p.G, H = p.H;

  if (threadIdx.x == 0) {
    if ((smem_u32(smem) & 1023u) != 0) atomicCAS(&g_error_flag, 0, 9);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(p_full, 8);
    mbar_init(pv_done, 1);
    mbar_init(o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  const int tok0 = p.tile_tok0[tile], ntok = p.tile_ntok[tile];      // fixed before the step began
  const int slot = p.tok_slot[tok0], pos0 = p.tok_pos[tok0];
  const int n_rows = ntok * G;
  const int key_hi = pos0 + ntok - 1;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kt_begin = key_lo / TILE_KEYS, kt_end = key_hi / TILE_KEYS + 1;
  rb_pdl_wait();                                           // q and the cache come from earlier kernels

  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // ---- Q rows into tensor memory: the A operand of S = Q K^T is read from there, so that the
  // MMAs fetch only K from shared memory.  Row r lives in lane r, two bfloat16 per column; the two
  // softmax threads of a row write half of it each (rows beyond n_rows are zero).
  if (warp >= 2) {
    const int quarter = warp & 3, half = (warp - 2) >> 2, r = quarter * 32 + lane;
    uint32_t w[D / 4];                                      // D/2 values = D/4 columns
    if (r < n_rows) {
      const int tok = tok0 + r / G, head = kvh * G + r % G;
      const uint4* src = reinterpret_cast<const uint4*>(p.q + ((int64_t)tok * H + head) * D + half * (D / 2));
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        const uint4 v = src[i];
        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < D / 4; ++i) w[i] = 0u;
    }
    const uint32_t q_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(Q_COL + half * (D / 4));
#pragma unroll
    for (int c = 0; c < D / 4; c += 16) tmem_st16(q_addr + c, w + c);
    tmem_st_wait();
  }
  if (warp >= 1) {                                         // the MMA warp waits for Q; the loader does not
    tcgen05_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS - 32) : "memory");
    tcgen05_fence_after();
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA loader
    if (lane == 0) {
      for (int kt = kt_begin, j = 0; kt < kt_end; ++kt, ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = ((j / KV_STAGES) & 1) ^ 1;
        int row[TILE_KEYS / PIECE];
#pragma unroll
        for (int h = 0; h < TILE_KEYS / PIECE; ++h) {      // a tile is two pieces of 64 positions
          const int key0 = kt * TILE_KEYS + h * PIECE;
          const int pi = min(key0 / p.page_size, p.max_pages - 1);       // past the sequence: any page, masked later
          const int page = p.page_table[(int64_t)slot * p.max_pages + pi];
          row[h] = (page * p.n_kv_heads + kvh) * p.page_size + key0 % p.page_size;
        }
        if (!mbar_wait(&k_empty[s], ph, 5)) break;
        mbar_expect_tx(&k_full[s], S::KV_TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
#pragma unroll
          for (int h = 0; h < TILE_KEYS / PIECE; ++h)
            tma_load_2d(smem + S::OFF_K + s * S::KV_TILE_BYTES + b * S::BLOCK + h * (PIECE * 128), &tmK, b * 64, row[h], &k_full[s]);
        if (!mbar_wait(&v_empty[s], ph, 5)) break;
        mbar_expect_tx(&v_full[s], S::KV_TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
#pragma unroll
          for (int h = 0; h < TILE_KEYS / PIECE; ++h)
            tma_load_2d(smem + S::OFF_V + s * S::KV_TILE_BYTES + b * S::BLOCK + h * (PIECE * 128), &tmV, b * 64, row[h], &v_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_mn(ROWS, TILE_KEYS, 0, 0);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc_mn(ROWS, D, 0, 1);           // P (K-major) x V (D contiguous)
      bool ok = true;
      const int n_tiles = kt_end - kt_begin;
      // S of tile j goes to S buffer j & 1.  S(j+1) is issued before P V (j), so the tensor cores
      // work on the next tile's scores while the softmax of this tile runs.
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES;
        if (!mbar_wait(&k_full[s], (j / KV_STAGES) & 1, 6)) return false;
        tcgen05_fence_after();
        const uint32_t k_addr = smem_u32(smem + S::OFF_K + s * S::KV_TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const uint64_t koff = (uint64_t)(k4 * 32 >> 4);
            // A: 16 values of Q = 8 columns of tensor memory; B: the keys' 16 values of block b
            umma_bf16_ts(tmem_base + (uint32_t)((j & 1) * TILE_KEYS), tmem_base + (uint32_t)(Q_COL + b * 32 + k4 * 8),
                         smem_desc_sw128(k_addr + b * S::BLOCK) + koff, idesc_s, (b > 0 || k4 > 0) ? 1u : 0u);
          }
        tcgen05_commit(&s_full[j & 1]);
        tcgen05_commit(&k_empty[s]);
        return true;
      };
      if (n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j % KV_STAGES;
        ok = mbar_wait(p_full, j & 1, 7);                    // P of this tile is in tensor memory
        if (!ok) break;
        ok = mbar_wait(&v_full[s], (j / KV_STAGES) & 1, 6);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t v_addr = smem_u32(smem + S::OFF_V + s * S::KV_TILE_BYTES);
#pragma unroll
        for (int k16 = 0; k16 < TILE_KEYS / 16; ++k16) {
          // A: 16 keys of P = 8 columns of tensor memory, in place of the S buffer of this tile;
          // B: 16 key rows of V (2048 bytes further per step), all D columns: 64-column blocks S::BLOCK apart
          umma_bf16_ts(tmem_base + O_COL, tmem_base + (uint32_t)((j & 1) * TILE_KEYS + k16 * 8),
                       smem_desc_sw128_mn(v_addr + k16 * 2048, S::BLOCK), idesc_o, (j > 0 || k16 > 0) ? 1u : 0u);
        }
        tcgen05_commit(&v_empty[s]);
        tcgen05_commit(pv_done);
      }
      tcgen05_commit(o_full);
    }
  } else {
    // ------------------------------------------------------------ softmax and output (warps 2..9)
    // Two threads per row: thread (quarter, lane, half) owns row quarter*32 + lane, the 64 keys
    // `half` of every tile and the columns [half*D/2, (half+1)*D/2) of O.  A wait that gives up sets
    // `failed`; the threads then stop waiting but keep the same control flow, so that the named
    // barrier below is always reached by all 256 of them.
    const int quarter = warp & 3;                            // the tensor-memory lanes a warp may touch: warp % 4
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool row_ok = r < n_rows;
    const int row_pos = pos0 + r / G;
    const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
    constexpr int HK = TILE_KEYS / 2;                        // keys per thread and tile
    constexpr int HD = D / 2;                                // columns of O per thread
    float m_run = -INFINITY, l_run = 0.f;
    bool failed = false;
    for (int kt = kt_begin, j = 0; kt < kt_end; ++kt, ++j) {
      bool ok = !failed;
      if (ok && lane == 0) ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, 8);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      failed |= !ok;
      tcgen05_fence_after();
      float sv[HK];
      const uint32_t s_addr = lane_addr + (uint32_t)((j & 1) * TILE_KEYS + half * HK);
#pragma unroll
      for (int c = 0; c < HK; c += 16) tmem_ld16(s_addr + c, reinterpret_cast<uint32_t*>(sv + c));
      tmem_ld_wait();
      const int key_base = kt * TILE_KEYS + half * HK;
      // a tile that every row of the CTA sees whole needs no mask (all tiles but those on the
      // diagonal and at the window's edge)
      const bool whole = kt * TILE_KEYS + TILE_KEYS - 1 <= pos0 &&
                         (p.window <= 0 || kt * TILE_KEYS >= max(0, key_hi - p.window + 1));
      float m_half;
      if (whole) {
        float t0 = sv[0], t1 = sv[1], t2 = sv[2], t3 = sv[3];          // four chains of three-input maxima
#pragma unroll
        for (int c = 4; c + 8 <= HK; c += 8) {
          t0 = max3(t0, sv[c], sv[c + 1]); t1 = max3(t1, sv[c + 2], sv[c + 3]);
          t2 = max3(t2, sv[c + 4], sv[c + 5]); t3 = max3(t3, sv[c + 6], sv[c + 7]);
        }
        t0 = max3(t0, sv[HK - 4], sv[HK - 3]); t1 = max3(t1, sv[HK - 2], sv[HK - 1]);
        m_half = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * p.scale_log2;   // the scale is positive
      } else {
        float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
        for (int c = 0; c < HK; c += 2) {
          const int key = key_base + c;
          sv[c] = (row_ok && key <= row_pos && key >= row_lo) ? sv[c] : -INFINITY;
          sv[c + 1] = (row_ok && key + 1 <= row_pos && key + 1 >= row_lo) ? sv[c + 1] : -INFINITY;
          t0 = fmaxf(t0, sv[c]); t1 = fmaxf(t1, sv[c + 1]);
        }
        m_half = fmaxf(t0, t1) * p.scale_log2;
      }
      // the row's max over both halves
      float* mx = row_max + (j & 1) * 2 * ROWS;
      mx[half * ROWS + r] = m_half;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const float m_new = fmaxf(m_run, fmaxf(m_half, mx[(half ^ 1) * ROWS + r]));
      // The exponent's reference m_run follows the true running max lazily: it moves only when the
      // max has grown by more than 8 (a factor 256 in P, harmless in bfloat16 and float32), so the
      // row of O in tensor memory is rescaled rarely.  l and O use the same reference, so O / l is exact.
      const bool moved = m_new > m_run + 8.0f || (m_run == -INFINITY && m_new > -INFINITY);
      const float m_next = moved ? m_new : m_run;
      const float m_use = m_next == -INFINITY ? 0.f : m_next;
      const float corr = moved ? exp2f(m_run - m_use) : 1.0f;      // exp2(-inf) = 0 before the first allowed key
      // P = 2^(S*scale - m), rounded to bfloat16, kept in registers until the P buffer is free
      uint32_t pw[HK / 2];
      {
        // packed pairs: one multiply-add and one add per two values, one exponential per value;
        // 2^(-inf) = 0 for masked keys
        const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg_m2 = pack2(-m_use, -m_use);
        uint64_t acc_a = pack2(0.f, 0.f), acc_b = acc_a;                 // four chains in two registers pairs
#pragma unroll
        for (int i = 0; i < HK / 2; i += 2) {
          float x0, x1, x2, x3;
          unpack2(fma2(pack2(sv[2 * i], sv[2 * i + 1]), scale2, neg_m2), x0, x1);
          unpack2(fma2(pack2(sv[2 * i + 2], sv[2 * i + 3]), scale2, neg_m2), x2, x3);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
          acc_a = add2(acc_a, pack2(p0, p1));
          acc_b = add2(acc_b, pack2(p2, p3));
          __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
          pw[i] = *reinterpret_cast<uint32_t*>(&h0);
          pw[i + 1] = *reinterpret_cast<uint32_t*>(&h1);
        }
        float s0, s1, s2, s3;
        unpack2(acc_a, s0, s1);
        unpack2(acc_b, s2, s3);
        const float sum = (s0 + s1) + (s2 + s3);
        l_run = l_run * corr + sum;
      }
      m_run = m_next;
      // P goes to tensor memory in place of this tile's S buffer (both threads of the row have
      // their S values in registers: they passed the barrier above).  The last reader of that
      // buffer, P V of tile j-2, is complete, since S of this tile was issued after it.  Only a
      // rescale of O has to wait, for P V of tile j-1.
      const bool rescale = j > 0 && __any_sync(0xffffffffu, moved);   // per warp: tensor-memory accesses are warp-wide
      if (rescale) {
        ok = !failed;
        if (ok && lane == 0) ok = mbar_wait(pv_done, (j - 1) & 1, 11);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        failed |= !ok;
        tcgen05_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD; c += 16) {
          uint32_t o[16];
          tmem_ld16(lane_addr + O_COL + half * HD + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tmem_st16(lane_addr + O_COL + half * HD + c, o);
        }
      }
      // 64 keys of this row = 32 columns of two bfloat16 each, at columns half*32 of the buffer
      const uint32_t p_addr = lane_addr + (uint32_t)((j & 1) * TILE_KEYS + half * (HK / 2));
#pragma unroll
      for (int c = 0; c < HK / 2; c += 16) tmem_st16(p_addr + c, pw + c);
      tmem_st_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- output: O / l, the sum l over both halves
    {
      bool ok = !failed;
      if (ok && lane == 0) ok = mbar_wait(o_full, 0, 10);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      failed |= !ok;
    }
    tcgen05_fence_after();
    row_max[half * ROWS + r] = l_run;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float l_all = l_run + row_max[(half ^ 1) * ROWS + r];
    if (!failed) {
      const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
      const int tok = tok0 + r / G, head = kvh * G + r % G;
      __nv_bfloat16* dst = p.out + ((int64_t)tok * H + head) * D + half * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 16) {
        uint32_t o[16];
        __syncwarp();
        tmem_ld16(lane_addr + O_COL + half * HD + c, o);
        tmem_ld_wait();
        if (row_ok) {
          uint32_t w[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int D>
int launch_tc(const CUtensorMap& tk, const CUtensorMap& tv, const TcAttnParams& p, int Kh, cudaStream_t stream) {
  auto kernel = attn_tc_kernel<D>;
  constexpr int smem = TcSmem<D>::BYTES;
  static RbOncePerDevice configured;
  if (configured.first()) {
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  }
  RB_LAUNCH("rb_attention_prefill_tc", (kernel), dim3(Kh, p.n_tiles), THREADS, smem, stream, tk, tv, p);
  return 0;
}

}  // namespace

#include "attention_decode_tma.cuh"

int rb_attention_combine(void* out, const float* part_o, const float* part_ml, int B, int H, int D, int n_splits,
                         cudaStream_t stream);   // attention_tiled.cu

// Whether the TMA-fed decode kernel takes these sizes (else rb_attention_decode).
RB_EXPORT int rb_attention_decode_tma_supports(int H, int Kh, int D, int page_size) {
  if (Kh <= 0 || H % Kh) return 0;
  return (D == 64 || D == 128) && page_size % decode_tma::TILE == 0 && H / Kh <= 16;
}

// The number of parts to cut the keys of a decode into, for `pairs` = sequences x kv heads, `tiles`
// 64-key tiles of the longest context and head size D.  When the pairs fit one wave of the
// three-stage kernel (two CTAs per SM at head size 128, four at 64): 1, 2, 4, 8 or 16, as many as
// still fit that wave; the parts of a pair are then a thread-block cluster and merge on chip (16
// where the device runs such clusters, else they are free CTAs with a merge kernel).  One when the
// pairs fit a wave of the two-stage kernel.  Else the count (up to 16) that fills whole such waves
// best; a second kernel merges those (clusters in a grid of several waves ran slower than free CTAs).
RB_EXPORT int rb_attention_decode_tma_parts(int pairs, int tiles, int D) {
  if (pairs <= 0 || tiles <= 0) return 1;
  const int deep = decode_tma::places(D, 3), shallow = decode_tma::places(D, 2) > deep ? decode_tma::places(D, 2) : deep;
  if (pairs <= deep) {
    int s = 1;
    while (s * 2 <= tiles && s < 16 && pairs * s * 2 <= deep) s *= 2;
    return s;
  }
  if (pairs <= shallow) return 1;
  const int most = tiles < 16 ? tiles : 16;
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= most; ++s) {
    const long long ctas = (long long)pairs * s;
    const double eff = (double)ctas / (double)(((ctas + shallow - 1) / shallow) * shallow);
    if (eff > best_eff + 0.02) { best = s; best_eff = eff; }
  }
  return best;
}

// Whether `parts` parts of `pairs` pairs merge on chip (no scratch, no second kernel): 2, 4, 8 or
// 16 parts in a grid that fits one wave of the three-stage kernel.
RB_EXPORT int rb_attention_decode_tma_on_chip(int pairs, int parts, int D) {
  if ((long long)pairs * parts > decode_tma::places(D, 3)) return 0;
  if (parts == 16) return decode_tma::cluster_of_16_runs() ? 1 : 0;
  return parts == 2 || parts == 4 || parts == 8;
}

// Decode: one token per sequence (batch row b is sequence b's token), keys and values by TMA.  With
// n_splits > 1, part_o [B, H, n_splits, D] and part_ml [B, H, n_splits, 2] float32 are scratch.
// cache_k / cache_v: [n_pages, Kh, page_size, D] bfloat16.
RB_EXPORT int rb_attention_decode_tma(void* out, const void* q, const void* cache_k, const void* cache_v,
                                      long long n_pages, const int* page_table, int max_pages, int page_size,
                                      const int* tok_pos, const int* tok_slot, int B, int H, int Kh, int D,
                                      float scale, int window, float* part_o, float* part_ml, int n_splits,
                                      cudaStream_t stream) {
  if (B == 0) return 0;
  RB_REQUIRE(rb_attention_decode_tma_supports(H, Kh, D, page_size),
             "rb_attention_decode_tma: sizes H=%d Kh=%d D=%d page=%d not supported", H, Kh, D, page_size);
  RB_REQUIRE(n_splits >= 1 && n_splits <= 65535 && B <= 2147483647, "rb_attention_decode_tma: n_splits %d", n_splits);
  // the parts are a thread-block cluster and merge on chip, or they leave their results in the
  // scratch and a second kernel merges them
  const bool cluster = rb_attention_decode_tma_on_chip(B * Kh, n_splits, D) != 0;
  RB_REQUIRE(n_splits == 1 || cluster || (part_o && part_ml), "rb_attention_decode_tma: split decode needs scratch");
  CUtensorMap tk, tv;
  const long long rows = n_pages * Kh * page_size;
  if (rb_get_tensor_map(&tk, cache_k, rows, D, D, decode_tma::TILE) != 0) return -1;
  if (rb_get_tensor_map(&tv, cache_v, rows, D, D, decode_tma::TILE) != 0) return -1;
  decode_tma::Params p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
  p.page_table = page_table; p.max_pages = max_pages; p.page_size = page_size; p.n_kv_heads = Kh;
  p.tok_pos = tok_pos; p.tok_slot = tok_slot; p.H = H; p.G = H / Kh;
  p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
  p.part_o = part_o; p.part_ml = part_ml; p.n_splits = n_splits; p.cluster = cluster ? 1 : 0;
  const int rc = D == 64 ? decode_tma::launch<64>(tk, tv, p, B, Kh, stream) : decode_tma::launch<128>(tk, tv, p, B, Kh, stream);
  if (rc != 0) return rc;
  if (n_splits > 1 && !cluster) return rb_attention_combine(out, part_o, part_ml, B, H, D, n_splits, stream);
  return 0;
}

int rb_attention_tc_error_flag(int* value, int reset) { return rb_file_error_flag(value, reset); }
int rb_attention_tc_error_flag_address(int** out) { return rb_file_error_flag_address(out); }

// Whether the tensor-memory prefill kernel takes these sizes.
RB_EXPORT int rb_attention_prefill_tc_supports(int H, int Kh, int D, int page_size) {
  if (Kh <= 0 || H % Kh) return 0;
  const int G = H / Kh;
  return (D == 64 || D == 128) && page_size % PIECE == 0 && G <= ROWS;
}

// Prefill over the paged cache: tile i covers tile_ntok[i] <= 128/G tokens of one sequence starting
// at batch row tile_tok0[i].  cache_k / cache_v: [n_pages, Kh, page_size, D] bfloat16.
RB_EXPORT int rb_attention_prefill_tc(void* out, const void* q, const void* cache_k, const void* cache_v,
                                      long long n_pages, const int* page_table, int max_pages, int page_size,
                                      const int* tok_pos, const int* tok_slot, const int* tile_tok0,
                                      const int* tile_ntok, int n_tiles, int H, int Kh, int D, float scale,
                                      int window, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  RB_REQUIRE(n_tiles <= 65535, "rb_attention_prefill_tc: %d tiles in one launch", n_tiles);
  RB_REQUIRE(rb_attention_prefill_tc_supports(H, Kh, D, page_size),
             "rb_attention_prefill_tc: sizes H=%d Kh=%d D=%d page=%d not supported", H, Kh, D, page_size);
  CUtensorMap tk, tv;
  const long long rows = n_pages * Kh * page_size;
  if (rb_get_tensor_map(&tk, cache_k, rows, D, D, PIECE) != 0) return -1;
  if (rb_get_tensor_map(&tv, cache_v, rows, D, D, PIECE) != 0) return -1;
  TcAttnParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
  p.page_table = page_table; p.max_pages = max_pages; p.page_size = page_size; p.n_kv_heads = Kh;
  p.tok_pos = tok_pos; p.tok_slot = tok_slot; p.tile_tok0 = tile_tok0; p.tile_ntok = tile_ntok; p.n_tiles = n_tiles;
  p.H = H; p.G = H / Kh; p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
  if (D == 64) return launch_tc<64>(tk, tv, p, Kh, stream);
  return launch_tc<128>(tk, tv, p, Kh, stream);
}
