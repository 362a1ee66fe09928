// Tiled attention over the paged cache for the bfloat16 path: prefill (many query rows per
// sequence) and decode (one token per sequence, keys split over several CTAs).
//
// One CTA works for ONE kv head of ONE sequence.  Its rows are (token, query head) pairs of the
// heads that share this kv head (row r -> token r / G, head kvh*G + r % G), so the G query heads
// of a group reuse every key and value the CTA loads.  Keys and values come in tiles of 64
// positions, which is one page (or an aligned part of a page) of the cache: a contiguous
// [64, D] block per kv head, fetched with cp.async into a double buffer.
//
// Per tile: S = Q K^T on mma.sync (bfloat16 in, float32 out); the score is (q.k)*scale with
// the scale folded into the exponent; causal and window masks by position; running max and sum
// in float32; P rounded to bfloat16 only as the operand of P V, accumulated in float32.
// crates/bitnet-core/src/llama/model.rs:260-289 (scores, mask by loop bound, P V), :102-114 (softmax).
//
// Prefill mode: 4 warps take 16 rows each and all 64 keys of a tile.  Decode mode: the rows are
// one token's G heads (G <= 16); the 4 warps take 16 keys each of every tile and are merged at
// the end; with n_splits > 1 each CTA covers a part of the sequence's tiles and writes an
// unnormalised partial (max, sum, O) that rb_attention_combine merges in split order.
#include "rb_common.cuh"

namespace {

constexpr int TILE_KEYS = 64;
constexpr int WARPS = 4;
constexpr int ROWS = 16 * WARPS;   // rows of a prefill CTA

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnParams {
  const __nv_bfloat16* q;   // [T, H, D]
  __nv_bfloat16* out;       // [T, H*D]
  RbPagedLayer cache;
  const int* tok_pos;
  const int* tok_slot;
  const int* tile_tok0;     // prefill: first token (row of the batch) of each tile
  const int* tile_ntok;     // prefill: tokens in each tile (same sequence, consecutive positions)
  int H, G;
  float scale_log2;         // scale * log2(e)
  int window;               // 0: none
  float* part_o;            // decode: [T, H, n_splits, D]
  float* part_ml;           // decode: [T, H, n_splits, 2]
  int n_splits;
};

// Row stride of the shared tiles: D values plus 8 of padding, so that the eight 16-byte rows an
// ldmatrix reads fall into different banks for every D that is a multiple of 16.
template <int D, bool DECODE> struct Smem {
  static constexpr int LD = D + 8;
  static constexpr int Q_ELEMS = (DECODE ? 16 : ROWS) * LD;     // decode: one token's heads only
  static constexpr int KV_ELEMS = TILE_KEYS * LD;
  // two stages of keys and values: one tile on its way while one is used.  (Three stages for
  // decode, with two CTAs per SM instead of three, measured the same at batch 8 and worse at 64.)
  static constexpr int STAGES = 2;
  static constexpr size_t BYTES = (size_t)(Q_ELEMS + 2 * STAGES * KV_ELEMS) * 2;
};

template <int D, bool DECODE>
__global__ void __launch_bounds__(WARPS * 32) attn_tiled_kernel(AttnParams p) {
  rb_pdl_launch_dependents();
  // The step's positions, slots and page tables were written before the step began, so they are
  // read at once; rb_pdl_wait() comes before the first access to what the kernel before this
  // one wrote (q, and the newest position's keys and values).
  using S = Smem<D, DECODE>;
  constexpr int LD = S::LD;
  constexpr int NT = DECODE ? 2 : 8;          // 8-key column tiles of S per warp
  constexpr int DT = D / 8;                   // 8-wide column tiles of O
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_bytes);
  __nv_bfloat16* sK = sQ + S::Q_ELEMS;        // [stages][64][LD]
  constexpr int NS = S::STAGES;
  __nv_bfloat16* sV = sK + NS * S::KV_ELEMS;  // [NS][64][LD] after the [NS][64][LD] of the keys

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int kvh = blockIdx.y;
  const int G = p.G, H = p.H;
  int tok0, ntok;
  if (DECODE) { tok0 = blockIdx.x; ntok = 1; } else { tok0 = p.tile_tok0[blockIdx.x]; ntok = p.tile_ntok[blockIdx.x]; }
  const int slot = p.tok_slot[tok0];
  const int pos0 = p.tok_pos[tok0];
  const int n_rows = ntok * G;
  const int key_hi = pos0 + ntok - 1;                                    // last key any row may see
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;      // first key any row may see
  int kt_begin = key_lo / TILE_KEYS, kt_end = key_hi / TILE_KEYS + 1;
  if (DECODE && p.n_splits > 1) {
    // the tiles are dealt evenly: part z takes [z*n/parts, (z+1)*n/parts), sizes that differ by at most one
    const int n = kt_end - kt_begin, z = blockIdx.z;
    kt_end = kt_begin + (int)((int64_t)(z + 1) * n / p.n_splits);
    kt_begin += (int)((int64_t)z * n / p.n_splits);
  }

  const __nv_bfloat16* Kbase = reinterpret_cast<const __nv_bfloat16*>(p.cache.k);
  const __nv_bfloat16* Vbase = reinterpret_cast<const __nv_bfloat16*>(p.cache.v);
  auto load_tile = [&](int kt, int buf) {
    const int key0 = kt * TILE_KEYS;
    const int page = p.cache.page_table[(int64_t)slot * p.cache.max_pages + key0 / p.cache.page_size];
    const int64_t off = (((int64_t)page * p.cache.n_kv_heads + kvh) * p.cache.page_size + key0 % p.cache.page_size) * D;
    const __nv_bfloat16* ksrc = Kbase + off;
    const __nv_bfloat16* vsrc = Vbase + off;
    __nv_bfloat16* kd = sK + buf * S::KV_ELEMS;
    __nv_bfloat16* vd = sV + buf * S::KV_ELEMS;
    for (int idx = threadIdx.x; idx < TILE_KEYS * (D / 8); idx += WARPS * 32) {
      const int r = idx / (D / 8), c = idx % (D / 8);
      cp_async16(kd + r * LD + c * 8, ksrc + r * D + c * 8);
      cp_async16(vd + r * LD + c * 8, vsrc + r * D + c * 8);
    }
  };

  // Decode: every tile but the one that holds the newest position was written by earlier steps,
  // so this CTA's first tile can be on its way before the wait.
  // Tiles are requested NS - 1 ahead; one commit group per tile (possibly empty), so that waiting
  // for all but the newest NS - 2 groups means the current tile has landed.
  const int newest = pos0 / TILE_KEYS;
  int n_early = 0;                     // tiles requested before the wait
  if (DECODE) {
    for (int i = 0; i < NS - 1; ++i) {
      const int kt = kt_begin + i;
      if (kt < kt_end && kt != newest && n_early == i) {
        load_tile(kt, i);
        cp_async_commit();
        n_early = i + 1;
      }
    }
  }
  rb_pdl_wait();

  // ---- Q rows into shared memory (rows beyond n_rows are zero)
  for (int idx = threadIdx.x; idx < ROWS * (D / 8); idx += WARPS * 32) {
    const int r = idx / (D / 8), c = idx % (D / 8);
    if (DECODE && r >= 16) break;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows) {
      const int tok = tok0 + r / G, head = kvh * G + r % G;
      v = *reinterpret_cast<const uint4*>(p.q + ((int64_t)tok * H + head) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
  }

  // ---- per-warp state
  const int rb = DECODE ? 0 : warp * 16;          // first row of this warp
  const int kw0 = DECODE ? warp * 16 : 0;         // first key of a tile this warp takes
  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // rows g and g+8 of this warp: their positions and validity
  int row_pos[2], row_lo[2];
  bool row_ok[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = rb + g + 8 * h;
    row_ok[h] = r < n_rows;
    row_pos[h] = pos0 + r / G;
    row_lo[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
  }

  for (int i = n_early; i < NS - 1; ++i) {        // the rest of the first NS - 1 tiles
    if (kt_begin + i < kt_end) load_tile(kt_begin + i, i);
    cp_async_commit();
  }
  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int buf = (kt - kt_begin) % NS;
    if (kt + NS - 1 < kt_end) load_tile(kt + NS - 1, (kt - kt_begin + NS - 1) % NS);
    cp_async_commit();
    cp_async_wait<NS - 1>();             // all but the newest NS - 1 groups: tile kt has landed
    __syncthreads();
    const __nv_bfloat16* tK = sK + buf * S::KV_ELEMS;
    const __nv_bfloat16* tV = sV + buf * S::KV_ELEMS;
    const int key_base = kt * TILE_KEYS + kw0;

    // a warp whose rows see none of this tile's keys skips it (prefill: tiles past the diagonal)
    const bool warp_has_rows = DECODE || rb < n_rows;
    const int warp_last_pos = DECODE ? pos0 : pos0 + min(n_rows - 1, rb + 15) / G;
    if (warp_has_rows && key_base <= warp_last_pos) {
      // ---- S = Q K^T
      float s[NT][4];
#pragma unroll
      for (int i = 0; i < NT; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, smem_addr(sQ + (rb + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          uint32_t b[4];
          // matrices: (keys nt*8.., d lo), (keys nt*8.., d hi), (keys (nt+1)*8.., d lo), (keys (nt+1)*8.., d hi)
          ldmatrix_x4(b, smem_addr(tK + (kw0 + nt * 8 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8));
          mma_bf16(s[nt], a, b[0], b[1]);
          mma_bf16(s[nt + 1], a, b[2], b[3]);
        }
      }
      // ---- mask, running max
      float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int h = c >> 1;
          const int key = key_base + nt * 8 + t4 * 2 + (c & 1);
          const bool ok = row_ok[h] && key <= row_pos[h] && key >= row_lo[h];
          const float v = ok ? s[nt][c] * p.scale_log2 : -INFINITY;
          s[nt][c] = v;
          m_new[h] = fmaxf(m_new[h], v);
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        m_use[h] = m_new[h] == -INFINITY ? 0.f : m_new[h];      // a row with nothing allowed so far
        corr[h] = exp2f(m_run[h] - m_use[h]);                    // exp2(-inf) = 0 on the first tile
        m_run[h] = m_new[h];
        l_run[h] *= corr[h];
      }
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
      // ---- P = exp2(S - m), row sums, P V
      uint32_t pa[NT / 2][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
        const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        pa[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
        pa[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int j = 0; j < NT / 2; ++j) {
#pragma unroll
        for (int dn = 0; dn < DT; dn += 2) {
          uint32_t b[4];
          // matrices: (keys 0-7, d dn), (keys 8-15, d dn), (keys 0-7, d dn+1), (keys 8-15, d dn+1)
          ldmatrix_x4_trans(b, smem_addr(tV + (kw0 + j * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + (dn + (lane >> 4)) * 8));
          mma_bf16(o[dn], pa[j], b[0], b[1]);
          mma_bf16(o[dn + 1], pa[j], b[2], b[3]);
        }
      }
    }
    __syncthreads();   // the other buffer is refilled at the top of the next round
  }

  // ---- row sums over the four threads of a quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  if (!DECODE) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rb + g + 8 * h;
      if (r >= n_rows) continue;
      const int tok = tok0 + r / G, head = kvh * G + r % G;
      const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
      __nv_bfloat16* dst = p.out + ((int64_t)tok * H + head) * D;
#pragma unroll
      for (int dn = 0; dn < DT; ++dn) {
        *reinterpret_cast<uint32_t*>(dst + dn * 8 + t4 * 2) = pack_bf16(o[dn][2 * h] * inv, o[dn][2 * h + 1] * inv);
      }
    }
    return;
  }

  // ---- decode: merge the four warps (each saw a quarter of every tile's keys)
  // shared layout (over the K/V buffers, free now): per warp [16 rows][D] O, then [16] m, [16] l
  float* mO = reinterpret_cast<float*>(sK);
  float* mM = mO + WARPS * 16 * D;
  float* mL = mM + WARPS * 16;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
#pragma unroll
    for (int dn = 0; dn < DT; ++dn) {
      mO[(warp * 16 + r) * D + dn * 8 + t4 * 2] = o[dn][2 * h];
      mO[(warp * 16 + r) * D + dn * 8 + t4 * 2 + 1] = o[dn][2 * h + 1];
    }
    if (t4 == 0) {
      mM[warp * 16 + r] = m_run[h];
      mL[warp * 16 + r] = l_run[h];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_rows * D; idx += WARPS * 32) {
    const int r = idx / D, d = idx % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, mM[w * 16 + r]);
    const float mu = m == -INFINITY ? 0.f : m;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float f = exp2f(mM[w * 16 + r] - mu);
      acc += mO[(w * 16 + r) * D + d] * f;
      l += mL[w * 16 + r] * f;
    }
    const int head = kvh * G + r;
    if (p.n_splits > 1) {
      const int64_t base = ((int64_t)tok0 * H + head) * p.n_splits + blockIdx.z;
      p.part_o[base * D + d] = acc;
      if (d == 0) { p.part_ml[base * 2] = m; p.part_ml[base * 2 + 1] = l; }
    } else {
      p.out[((int64_t)tok0 * H + head) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
  }
}

// Merges the partials of a split decode in split order.
__global__ void attn_combine_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, int n_splits, int D) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  // One thread per output value.  The parts are taken 16 at a time with all their loads issued
  // before the first use, so that a merge of up to 16 parts waits for memory once.
  const int64_t th = blockIdx.x;   // token * H + head
  const int d = threadIdx.x;
  if (d >= D) return;
  const float* ml = part_ml + th * n_splits * 2;
  const float* po = part_o + th * n_splits * D + d;
  float m_run = -INFINITY, l_run = 0.f, acc = 0.f;
  for (int s0 = 0; s0 < n_splits; s0 += 16) {
    float m[16], l[16], o[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const bool have = s0 + i < n_splits;
      m[i] = have ? ml[(s0 + i) * 2] : -INFINITY;
      l[i] = have ? ml[(s0 + i) * 2 + 1] : 0.f;
      o[i] = have ? po[(int64_t)(s0 + i) * D] : 0.f;
    }
    float mg = m_run;
#pragma unroll
    for (int i = 0; i < 16; ++i) mg = fmaxf(mg, m[i]);
    const float mu = mg == -INFINITY ? 0.f : mg;
    const float keep = exp2f(m_run - mu);          // 0 for the first group
    l_run *= keep;
    acc *= keep;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float w = exp2f(m[i] - mu);            // 0 for a part without keys and beyond the last part
      l_run += l[i] * w;
      acc += o[i] * w;
    }
    m_run = mg;
  }
  out[th * D + d] = __float2bfloat16_rn(l_run > 0.f ? acc / l_run : 0.f);
}

template <int D, bool DECODE>
int launch_one(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  auto kernel = attn_tiled_kernel<D, DECODE>;
  size_t smem = Smem<D, DECODE>::BYTES;
  if (DECODE) {
    const size_t merge = (size_t)(WARPS * 16 * D + 2 * WARPS * 16) * 4;
    const size_t kv = (size_t)2 * Smem<D, DECODE>::STAGES * Smem<D, DECODE>::KV_ELEMS * 2;
    if (merge > kv) smem += merge - kv;
  }
  static RbOncePerDevice configured;
  if (configured.first()) {
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  RB_LAUNCH("kernel", (kernel), grid, WARPS * 32, smem, stream, p);
  RB_CHECK_LAUNCH("rb_attention_tiled");
  return 0;
}

template <bool DECODE>
int launch_d(int D, const AttnParams& p, dim3 grid, cudaStream_t stream) {
  switch (D) {
    case 16: return launch_one<16, DECODE>(p, grid, stream);
    case 32: return launch_one<32, DECODE>(p, grid, stream);
    case 48: return launch_one<48, DECODE>(p, grid, stream);
    case 64: return launch_one<64, DECODE>(p, grid, stream);
    case 80: return launch_one<80, DECODE>(p, grid, stream);
    case 96: return launch_one<96, DECODE>(p, grid, stream);
    case 112: return launch_one<112, DECODE>(p, grid, stream);
    case 128: return launch_one<128, DECODE>(p, grid, stream);
    case 160: return launch_one<160, DECODE>(p, grid, stream);
    case 192: return launch_one<192, DECODE>(p, grid, stream);
    case 256: return launch_one<256, DECODE>(p, grid, stream);
  }
  RB_FAIL("rb_attention_tiled: head_dim %d is not built (16..128 in steps of 16, 160, 192, 256)", D);
}

}  // namespace

// Whether the tiled kernel takes these sizes (the caller uses the plain kernel otherwise).
RB_EXPORT int rb_attention_tiled_supports(int H, int Kh, int D, int page_size, int decode) {
  if (Kh <= 0 || H % Kh) return 0;
  const int G = H / Kh;
  const bool d_ok = (D % 16 == 0 && D >= 16 && D <= 128) || D == 160 || D == 192 || D == 256;
  if (!d_ok || page_size % TILE_KEYS) return 0;
  if (decode) return G <= 16;
  return G <= ROWS;
}

// Prefill: n_tiles tiles of tokens; tile i covers tile_ntok[i] <= 64/G tokens of one sequence
// starting at batch row tile_tok0[i].
RB_EXPORT int rb_attention_prefill(void* out, const void* q, const void* cache_k, const void* cache_v,
                                   const int* page_table, int max_pages, int page_size, const int* tok_pos,
                                   const int* tok_slot, const int* tile_tok0, const int* tile_ntok, int n_tiles,
                                   int H, int Kh, int D, float scale, int window, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  RB_REQUIRE(rb_attention_tiled_supports(H, Kh, D, page_size, 0), "rb_attention_prefill: sizes H=%d Kh=%d D=%d page=%d not supported", H, Kh, D, page_size);
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
  p.cache = RbPagedLayer{(void*)cache_k, (void*)cache_v, page_table, max_pages, page_size, Kh, D};
  p.tok_pos = tok_pos; p.tok_slot = tok_slot; p.tile_tok0 = tile_tok0; p.tile_ntok = tile_ntok;
  p.H = H; p.G = H / Kh; p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
  p.part_o = nullptr; p.part_ml = nullptr; p.n_splits = 1;
  return launch_d<false>(D, p, dim3(n_tiles, Kh, 1), stream);
}

// Parts a decode's keys are cut into for rb_attention_decode.  About three CTAs of the decode kernel
// fit an SM; the number of parts is the one (up to 16) that fills whole waves of those places best,
// since a last wave with a few CTAs costs as much as a full one.
RB_EXPORT int rb_attention_decode_parts(int batch, int n_kv_heads, int max_context) {
  const int tiles = max_context > 0 ? (max_context + TILE_KEYS - 1) / TILE_KEYS : 1;
  const long long places = 3ll * rb_sm_count(), pairs = (long long)batch * n_kv_heads;
  if (pairs <= 0) return 1;
  const int most = tiles < 16 ? tiles : 16;
  if (pairs <= places) {                       // one wave: as many parts as fit it
    const long long fit = places / pairs;
    return (int)(fit < most ? (fit < 1 ? 1 : fit) : most);
  }
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= most; ++s) {
    const long long ctas = pairs * s;
    const double eff = (double)ctas / (double)(((ctas + places - 1) / places) * places);
    if (eff > best_eff + 0.02) { best = s; best_eff = eff; }
  }
  return best;
}

// Merges the partials of a split decode (also for the TMA-fed decode kernel, which lives in another file).
int rb_attention_combine(void* out, const float* part_o, const float* part_ml, int B, int H, int D, int n_splits,
                         cudaStream_t stream) {
  RB_LAUNCH("attn_combine_kernel", (attn_combine_kernel), B * H, (D + 31) / 32 * 32, 0, stream, (__nv_bfloat16*)out, part_o, part_ml, n_splits, D);
  RB_CHECK_LAUNCH("rb_attention_combine");
  return 0;
}

// Decode: one token per sequence (batch row b is sequence b's token).  With n_splits > 1,
// part_o [B, H, n_splits, D] and part_ml [B, H, n_splits, 2] float32 are scratch.
RB_EXPORT int rb_attention_decode(void* out, const void* q, const void* cache_k, const void* cache_v,
                                  const int* page_table, int max_pages, int page_size, const int* tok_pos,
                                  const int* tok_slot, int B, int H, int Kh, int D, float scale, int window,
                                  float* part_o, float* part_ml, int n_splits, cudaStream_t stream) {
  if (B == 0) return 0;
  RB_REQUIRE(rb_attention_tiled_supports(H, Kh, D, page_size, 1), "rb_attention_decode: sizes H=%d Kh=%d D=%d page=%d not supported", H, Kh, D, page_size);
  RB_REQUIRE(n_splits >= 1 && n_splits <= 65535, "rb_attention_decode: n_splits %d", n_splits);
  RB_REQUIRE(n_splits == 1 || (part_o && part_ml), "rb_attention_decode: split decode needs scratch");
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
  p.cache = RbPagedLayer{(void*)cache_k, (void*)cache_v, page_table, max_pages, page_size, Kh, D};
  p.tok_pos = tok_pos; p.tok_slot = tok_slot; p.tile_tok0 = nullptr; p.tile_ntok = nullptr;
  p.H = H; p.G = H / Kh; p.scale_log2 = scale * 1.4426950408889634f; p.window = window;
  p.part_o = part_o; p.part_ml = part_ml; p.n_splits = n_splits;
  if (launch_d<true>(D, p, dim3(B, Kh, n_splits), stream) != 0) return -1;
  if (n_splits > 1) return rb_attention_combine(out, part_o, part_ml, B, H, D, n_splits, stream);
  return 0;
}

// ---------------------------------------------------------------- decode without caller scratch
// See rb_no_alloc.h.  The scratch of the split decode lives in this file-scope device array.
// In host code its name is only a handle for the runtime, not a device address; the address
// each device maps it to is looked up once per device and that pointer goes to the kernels.
#include "rb_no_alloc.h"
#include <mutex>

static __device__ __align__(256) float g_static_scratch[RB_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_ptr[MAX_DEVICES] = {nullptr};
std::mutex g_static_scratch_mutex;

// Device address of the static scratch on the current device (set up at the first call there).
int static_scratch(float** ptr) {
  int dev = -1;
  RB_CUDA(cudaGetDevice(&dev));
  RB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "rb_attention_decode_static: device %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    RB_CUDA(cudaGetSymbolAddress((void**)&p, g_static_scratch));
    RB_REQUIRE(p != nullptr, "rb_attention_decode_static: no device address for the static scratch");
    g_static_scratch_ptr[dev] = p;
  }
  *ptr = g_static_scratch_ptr[dev];
  return 0;
}
}  // namespace

RB_EXPORT int rb_attention_decode_static(void* out, const void* q, const void* cache_k, const void* cache_v,
                                         const int* page_table, int max_pages, int page_size, const int* tok_pos,
                                         const int* tok_slot, int B, int H, int Kh, int D, float scale, int window,
                                         int n_splits, cudaStream_t stream) {
  if (B == 0) return 0;
  RB_REQUIRE(B > 0 && H > 0 && D > 0 && n_splits >= 1, "rb_attention_decode_static: bad sizes B=%d H=%d D=%d splits=%d",
             B, H, D, n_splits);
  // one part: the kernel writes the output itself and no scratch is used, whatever the sizes
  const long long need = n_splits > 1 ? (long long)B * H * n_splits * (D + 2) : 0;
  RB_REQUIRE(need <= (long long)RB_STATIC_SCRATCH_FLOATS,
             "rb_attention_decode_static: B*H*n_splits*(D+2) = %lld float32 values of scratch exceed the static "
             "array's %d; use fewer splits or rb_attention_decode with caller scratch",
             need, (int)RB_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  if (static_scratch(&scratch) != 0) return -1;
  float* part_o = scratch;                                       // [B, H, n_splits, D]
  float* part_ml = scratch + (size_t)B * H * n_splits * D;       // [B, H, n_splits, 2]
  return rb_attention_decode(out, q, cache_k, cache_v, page_table, max_pages, page_size, tok_pos, tok_slot, B, H,
                             Kh, D, scale, window, part_o, part_ml, n_splits, stream);
}

RB_CHECK_READER(attention_tiled)
