// Decode attention (one token per sequence) with keys and values brought in by TMA.
//
// The arithmetic is that of the decode mode of attention_tiled.cu: one CTA works for ONE kv head of
// ONE sequence on a part of its keys; its rows are the token's G query heads (G <= 16, padded to the
// 16 rows of mma.sync m16n8k16); keys and values come in tiles of 64 positions, of which each of the
// four warps takes 16 keys; the warps are merged at the end.  When the keys are not split the CTA
// writes the result itself.  When they are, the parts of a (sequence, kv head) are either a
// thread-block cluster (2, 4, 8 or 16 CTAs of a grid that runs as one wave) that merges through
// distributed shared memory, or free CTAs that write unnormalised partials (max, sum, O) for
// attn_combine_kernel.  crates/bitnet-core/src/llama/model.rs:260-289 (scores, mask by loop bound,
// P V), :102-114.
//
// What differs is how a tile gets into shared memory.  There, every thread issues 32 cp.async of 16
// bytes per tile, which costs the four warps about a third of a tile's time; here one thread asks
// for a tile with 2 * D/64 TMA boxes of [64 positions, 64 values] (128-byte swizzle, the layout
// ldmatrix reads without bank conflicts) and everybody waits on the stage's mbarrier.  Head sizes 64
// and 128.  This header is included by attention_tcgen05.cu, whose TMA and mbarrier helpers and
// error word it shares; every wait is bounded.
#pragma once

namespace decode_tma {

constexpr int TILE = 64;           // positions per tile = per TMA box
constexpr int WARPS_D = 4;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2bf(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct Params {
  const __nv_bfloat16* q;   // [B, H, D]
  __nv_bfloat16* out;       // [B, H*D]
  const int* page_table;
  int max_pages, page_size, n_kv_heads;
  const int* tok_pos;
  const int* tok_slot;
  int H, G;
  float scale_log2;         // scale * log2(e)
  int window;               // 0: none
  float* part_o;            // [B, H, n_splits, D]
  float* part_ml;           // [B, H, n_splits, 2]
  int n_splits;
  int cluster;              // 1: the parts of a (sequence, kv head) are a thread-block cluster and merge on chip
};

// NS: stages of keys and values.  Two stages let three CTAs share an SM, three stages two: the
// launcher takes three when the whole grid fits two CTAs per SM at once (a small batch), where one
// more tile in flight per CTA counts for more than a third CTA, and two otherwise.
template <int D, int NS> struct Smem {
  static constexpr int DB = D / 64;                      // 64-value blocks of a head
  static constexpr int BLOCK = TILE * 128;               // [64 positions][128 bytes]
  static constexpr int TILE_BYTES = DB * BLOCK;          // keys (or values) of one tile
  static constexpr int LDQ = D + 8;                      // row stride of Q (padded against bank conflicts)
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = NS * TILE_BYTES;
  static constexpr int OFF_Q = 2 * NS * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_Q + 16 * LDQ * 2;
  static constexpr int KV_BYTES = 2 * NS * TILE_BYTES;
  // the merge of the four warps reuses the tile buffers: [4 warps][16 rows][D] floats, then max and sum
  static constexpr int MERGE_BYTES = (WARPS_D * 16 * D + 2 * WARPS_D * 16) * 4;
  // behind it, what this CTA shows the other parts of its cluster: [16 rows][D] floats, max and sum
  static constexpr int SHOW_BYTES = (16 * D + 2 * 16) * 4;
  static_assert(MERGE_BYTES + SHOW_BYTES <= OFF_Q, "the merge areas lie inside the tile buffers");
  static constexpr int BYTES = (MERGE_BYTES > OFF_BAR ? MERGE_BYTES : OFF_BAR) + 64 + 1024;   // + room to align
};

// byte offset of element (row, col) of a tile: 64-value blocks of [64 rows][128 bytes] whose
// 16-byte chunks are exchanged by the row's low three bits (the 128-byte swizzle of the TMA box)
template <int D> __device__ __forceinline__ uint32_t tile_off(int row, int col) {
  return (uint32_t)((col >> 6) * (TILE * 128) + row * 128 + (((((col & 63) >> 3) ^ (row & 7))) << 4) + (col & 7) * 2);
}

template <int D, int NS>
__global__ void __launch_bounds__(WARPS_D * 32) attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmV, Params p) {
  rb_pdl_launch_dependents();
  using S = Smem<D, NS>;
  constexpr int DB = S::DB, LDQ = S::LDQ;
  constexpr int NT = 2;                       // 8-key column tiles of S per warp (16 keys)
  constexpr int DT = D / 8;                   // 8-wide column tiles of O
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem + S::OFF_Q);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (S::MERGE_BYTES > S::OFF_BAR ? S::MERGE_BYTES : S::OFF_BAR));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int kvh = blockIdx.y, tok0 = blockIdx.x;
  const int G = p.G, H = p.H;
  // positions, slots and page tables were written before the step began: they are read at once
  const int slot = p.tok_slot[tok0];
  const int pos0 = p.tok_pos[tok0];
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  int kt_begin = key_lo / TILE, kt_end = pos0 / TILE + 1;
  if (p.n_splits > 1) {
    // the tiles are dealt evenly: part z takes [z*n/parts, (z+1)*n/parts), sizes that differ by at most one
    const int n = kt_end - kt_begin, z = blockIdx.z;
    kt_end = kt_begin + (int)((int64_t)(z + 1) * n / p.n_splits);
    kt_begin += (int)((int64_t)z * n / p.n_splits);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // one thread asks for a tile: keys and values of 64 positions of this kv head, D/64 boxes each
  auto request = [&](int kt, int buf) {
    const int key0 = kt * TILE;
    const int page = p.page_table[(int64_t)slot * p.max_pages + key0 / p.page_size];
    const int row = (page * p.n_kv_heads + kvh) * p.page_size + key0 % p.page_size;
    mbar_expect_tx(&full[buf], 2 * S::TILE_BYTES);
#pragma unroll
    for (int b = 0; b < DB; ++b) {
      tma_load_2d(smem + S::OFF_K + buf * S::TILE_BYTES + b * S::BLOCK, &tmK, b * 64, row, &full[buf]);
      tma_load_2d(smem + S::OFF_V + buf * S::TILE_BYTES + b * S::BLOCK, &tmV, b * 64, row, &full[buf]);
    }
  };
  // Every tile but the one that holds the newest position was written by earlier steps, so this
  // CTA's first tile can be on its way before the wait for the kernel that wrote the newest.
  const int newest = pos0 / TILE;
  int n_early = 0;                     // tiles requested before the wait (thread 0's count)
  if (threadIdx.x == 0) {
    for (int i = 0; i < NS - 1; ++i)
      if (kt_begin + i < kt_end && kt_begin + i != newest && n_early == i) {
        request(kt_begin + i, i);
        n_early = i + 1;
      }
  }
  rb_pdl_wait();

  // ---- the token's G query rows into shared memory (rows beyond G are zero)
  for (int idx = threadIdx.x; idx < 16 * (D / 8); idx += WARPS_D * 32) {
    const int r = idx / (D / 8), c = idx % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) v = *reinterpret_cast<const uint4*>(p.q + ((int64_t)tok0 * H + kvh * G + r) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * LDQ + c * 8) = v;
  }
  if (threadIdx.x == 0)
    for (int i = n_early; i < NS - 1; ++i)        // the rest of the first NS - 1 tiles
      if (kt_begin + i < kt_end) request(kt_begin + i, i);

  // ---- per-warp state: all 16 rows, keys kw0 .. kw0+15 of every tile
  const int kw0 = warp * 16;
  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const bool row_ok[2] = {g < G, g + 8 < G};
  const uint32_t q_base = smem_u32(sQ);
  bool failed = false;
  __syncthreads();                       // Q is in shared memory

  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int i = kt - kt_begin, buf = i % NS;
    // the tile NS - 1 ahead goes into the stage that everybody left at the end of the last round
    if (threadIdx.x == 0 && kt + NS - 1 < kt_end) request(kt + NS - 1, (i + NS - 1) % NS);
    if (!failed && !mbar_wait(&full[buf], (uint32_t)((i / NS) & 1), 14)) failed = true;
    const uint32_t tK = smem_u32(smem + S::OFF_K + buf * S::TILE_BYTES);
    const uint32_t tV = smem_u32(smem + S::OFF_V + buf * S::TILE_BYTES);
    const int key_base = kt * TILE + kw0;
    if (key_base <= pos0) {
      // ---- S = Q K^T: two accumulators per 8-key tile, over even and odd steps of d, so that the
      // chain of dependent products is half as long
      float s[NT][4], s2[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; s2[n][0] = s2[n][1] = s2[n][2] = s2[n][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4], b[4];
        ldsm_x4(a, q_base + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * LDQ + kk * 16 + (lane >> 4) * 8) * 2);
        // matrices: (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
        ldsm_x4(b, tK + tile_off<D>(kw0 + (lane >> 4) * 8 + (lane & 7), kk * 16 + ((lane >> 3) & 1) * 8));
        if (kk & 1) { mma16816(s2[0], a, b[0], b[1]); mma16816(s2[1], a, b[2], b[3]); }
        else { mma16816(s[0], a, b[0], b[1]); mma16816(s[1], a, b[2], b[3]); }
      }
      // ---- mask, running max
      float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int h = c >> 1;
          const int key = key_base + n * 8 + t4 * 2 + (c & 1);
          const bool ok = row_ok[h] && key <= pos0 && key >= key_lo;
          const float v = ok ? (s[n][c] + s2[n][c]) * p.scale_log2 : -INFINITY;
          s[n][c] = v;
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
      for (int d = 0; d < DT; ++d) {
        o[d][0] *= corr[0]; o[d][1] *= corr[0];
        o[d][2] *= corr[1]; o[d][3] *= corr[1];
      }
      // ---- P = exp2(S - m), row sums, P V
      uint32_t pa[4];
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float p0 = exp2f(s[n][0] - m_use[0]), p1 = exp2f(s[n][1] - m_use[0]);
        const float p2 = exp2f(s[n][2] - m_use[1]), p3 = exp2f(s[n][3] - m_use[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        pa[n * 2 + 0] = pack2bf(p0, p1);
        pa[n * 2 + 1] = pack2bf(p2, p3);
      }
#pragma unroll
      for (int dn = 0; dn < DT; dn += 2) {
        uint32_t b[4];
        // matrices: (keys 0-7, d dn), (keys 8-15, d dn), (keys 0-7, d dn+1), (keys 8-15, d dn+1)
        ldsm_x4_trans(b, tV + tile_off<D>(kw0 + ((lane >> 3) & 1) * 8 + (lane & 7), (dn + (lane >> 4)) * 8));
        mma16816(o[dn], pa, b[0], b[1]);
        mma16816(o[dn + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();   // everybody has left this stage: the round after next may refill it
  }

  // ---- row sums over the four threads of a quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  // ---- merge the four warps (each saw a quarter of every tile's keys), over the tile buffers,
  // which are free: every request has been waited for
  float* mO = reinterpret_cast<float*>(smem);
  float* mM = mO + WARPS_D * 16 * D;
  float* mL = mM + WARPS_D * 16;
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
  if (failed && !p.cluster) return;
  // what the other parts of the cluster read: this part's sums, maximum and normaliser per row
  float* sO = reinterpret_cast<float*>(smem + S::MERGE_BYTES);
  float* sM = sO + 16 * D;
  float* sL = sM + 16;
  if (!failed) {
    for (int idx = threadIdx.x; idx < G * D; idx += WARPS_D * 32) {
      const int r = idx / D, d = idx % D;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS_D; ++w) m = fmaxf(m, mM[w * 16 + r]);
      const float mu = m == -INFINITY ? 0.f : m;
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS_D; ++w) {
        const float f = exp2f(mM[w * 16 + r] - mu);
        acc += mO[(w * 16 + r) * D + d] * f;
        l += mL[w * 16 + r] * f;
      }
      const int head = kvh * G + r;
      if (p.cluster) {
        sO[r * D + d] = acc;
        if (d == 0) { sM[r] = m; sL[r] = l; }
      } else if (p.n_splits > 1) {
        const int64_t base = ((int64_t)tok0 * H + head) * p.n_splits + blockIdx.z;
        p.part_o[base * D + d] = acc;
        if (d == 0) { p.part_ml[base * 2] = m; p.part_ml[base * 2 + 1] = l; }
      } else {
        p.out[((int64_t)tok0 * H + head) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
      }
    }
  }
  if (!p.cluster) return;
  // ---- the parts of this (sequence, kv head) are one cluster: every CTA finishes a share of the
  // output values from all parts, read through distributed shared memory and merged in part
  // order.  Every thread of every CTA passes both barriers, also after a wait that gave up.
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (!failed) {
    uint32_t my;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(my));
    const int parts = p.n_splits;                 // 2, 4, 8 or 16
    for (int idx = (int)my * WARPS_D * 32 + threadIdx.x; idx < G * D; idx += parts * WARPS_D * 32) {
      const int r = idx / D, d = idx % D;
      float m[16], l[16], o[16];
#pragma unroll
      for (int z = 0; z < 16; ++z) {              // all loads first
        m[z] = -INFINITY; l[z] = 0.f; o[z] = 0.f;
        if (z < parts) {
          uint32_t am, al, ao;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(am) : "r"(smem_u32(sM + r)), "r"((uint32_t)z));
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(al) : "r"(smem_u32(sL + r)), "r"((uint32_t)z));
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ao) : "r"(smem_u32(sO + r * D + d)), "r"((uint32_t)z));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(m[z]) : "r"(am));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(l[z]) : "r"(al));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(o[z]) : "r"(ao));
        }
      }
      float mg = -INFINITY;
#pragma unroll
      for (int z = 0; z < 16; ++z) mg = fmaxf(mg, m[z]);
      const float mu = mg == -INFINITY ? 0.f : mg;
      float acc = 0.f, ls = 0.f;
#pragma unroll
      for (int z = 0; z < 16; ++z) {
        const float w = exp2f(m[z] - mu);          // 0 for a part without keys and beyond the last part
        ls += l[z] * w;
        acc += o[z] * w;
      }
      p.out[((int64_t)tok0 * H + kvh * G + r) * D + d] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
    }
  }
  // nobody's shared memory goes away while another part reads it
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int D, int NS>
int launch_ns(const CUtensorMap& tk, const CUtensorMap& tv, const Params& p, int B, int Kh, cudaStream_t stream) {
  auto kernel = attn_decode_tma_kernel<D, NS>;
  constexpr int smem = Smem<D, NS>::BYTES;
  static RbOncePerDevice configured;
  if (configured.first()) {
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  }
  if (p.cluster) {
    static RbOncePerDevice large_allowed;
    if (p.n_splits > 8 && large_allowed.first()) {      // clusters of more than 8 CTAs have to be asked for
      RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(B, Kh, p.n_splits);
    cfg.blockDim = dim3(WARPS_D * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = p.n_splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = rb_pdl_enabled() ? 2 : 1;
    RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, tk, tv, p));
    return 0;
  }
  RB_LAUNCH("rb_attention_decode_tma", (kernel), dim3(B, Kh, p.n_splits), WARPS_D * 32, smem, stream, tk, tv, p);
  return 0;
}

// CTAs of the kernel with `stages` stages that run together: what shared memory lets an SM hold
// (227 KB, 1 KB of it per CTA for the system), at most 4 (128 threads of up to 128 registers).
// Head size 128: 2 per SM with three stages, 3 with two.  Head size 64: 4 either way.
inline int places(int D, int stages) {
  const int sms = rb_sm_count();
  const int bytes = D == 64 ? (stages == 3 ? Smem<64, 3>::BYTES : Smem<64, 2>::BYTES)
                            : (stages == 3 ? Smem<128, 3>::BYTES : Smem<128, 2>::BYTES);
  int per_sm = (227 * 1024) / (bytes + 1024);
  if (per_sm > 4) per_sm = 4;
  return sms * per_sm;
}

// Whether clusters of 16 CTAs of the three-stage kernel can run on this device (asked once).
inline bool cluster_of_16_runs() {
  static int answer = -1;
  if (answer < 0) {
    answer = 0;
    auto kernel = attn_decode_tma_kernel<128, 3>;
    constexpr int smem = Smem<128, 3>::BYTES;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(1, 1, 16);
      cfg.blockDim = dim3(WARPS_D * 32, 1, 1);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 16;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n >= 1) answer = 1;
    }
    (void)cudaGetLastError();      // a refusal above is an answer, not an error of a later launch
  }
  return answer == 1;
}

template <int D>
int launch(const CUtensorMap& tk, const CUtensorMap& tv, const Params& p, int B, int Kh, cudaStream_t stream) {
  // the deeper ring when the whole grid runs at once with it, or when the shallower one holds no more CTAs
  if ((long long)B * Kh * p.n_splits <= places(D, 3) || places(D, 2) <= places(D, 3))
    return launch_ns<D, 3>(tk, tv, p, B, Kh, stream);
  return launch_ns<D, 2>(tk, tv, p, B, Kh, stream);
}

}  // namespace decode_tma
