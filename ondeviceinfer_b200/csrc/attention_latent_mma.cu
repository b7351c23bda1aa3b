// bf16 causal attention over a paged cache of shared rows (a cached row is key and value at once: the value is
// its first DV lanes; every query head reads the same row), on the tensor cores: mma.sync m16n8k16 with fp32
// accumulation, the softmax in fp32 (running maximum, base 2).  It is the attention of a latent cache for single
// tokens and for portions of prompts; rows are far wider than a head (hundreds of lanes), so the partition differs
// from the kernels for ordinary heads: a block owns 16 query rows, its four warps split a tile's 64 keys for the
// scores and the value lanes for the output, and the tile's weights pass through shared memory.
//
// Compile with -DODI_HEAD_DIM=<row width D, a multiple of 16 up to 1024> -DODI_VALUE_DIM=<DV, a multiple of 16, at
// most D and 512>.  Pages hold 64 positions.
//
// Work item: one sequence, a tile of query rows -- `bq` consecutive tokens times up to 16 query heads -- and, when
// the key range is split, one split.  Key j is visible to the query at position p iff j <= p and (window == 0 or
// j > p - window).  With splits > 1 every split writes an un-normalised partial (acc[DV], maximum in natural-log
// units, sum) and the combine kernel merges them in split order.
#include "common.cuh"

#ifndef ODI_HEAD_DIM
#error "compile with -DODI_HEAD_DIM=<row width> -DODI_VALUE_DIM=<value width>"
#endif
#ifndef ODI_VALUE_DIM
#error "compile with -DODI_VALUE_DIM=<value width>"
#endif
#define D ODI_HEAD_DIM
#define DV ODI_VALUE_DIM
static_assert(D % 16 == 0 && D >= 16 && D <= 1024, "row widths in steps of 16 up to 1024");
static_assert(DV % 16 == 0 && DV >= 16 && DV <= 512 && DV <= D, "value widths in steps of 16 up to 512, within the row");

#define KT 64                        // keys per tile
#define PAGE 64                      // positions per page (a tile never crosses a page)
#define WARPS 4
#define ROWS 16                      // query rows per block
#define ROWB (2 * D + 16)            // bytes per shared-memory row of a key tile and of the query tile
#define K_BYTES (KT * ROWB)
#define Q_BYTES (ROWS * ROWB)
#define P_ROWB (2 * KT + 16)         // bytes per row of the weights
#define P_BYTES (ROWS * P_ROWB)
#define STAT_BYTES (2 * WARPS * ROWS * 4)
#define STAGES ((Q_BYTES + 2 * K_BYTES + P_BYTES + STAT_BYTES) <= 220 * 1024 ? 2 : 1)
#define SMEM_BYTES (Q_BYTES + STAGES * K_BYTES + P_BYTES + STAT_BYTES)
#define KSTEPS (D / 16)
#define UNITS (DV / 16)              // value lanes in units of 16
#define UPW ((UNITS + WARPS - 1) / WARPS)   // units per warp (warp w owns units w, w + 4, ...)
#define LOG2E 1.4426950408889634f
#define LN2 0.6931471805599453f

struct LatentAttnArgs {
  const bf16* q;          // [n_tokens, nq, D]
  const bf16* pool;       // [pages, 64, D]
  bf16* out;              // [n_tokens, nq * DV]
  float* partial;         // [n_tokens, nq, splits, DV + 2] when splits > 1
  const int* cu_q;        // [n_seqs + 1]
  const int* past;        // [n_seqs]
  const int* page_start;
  const int* page_ids;
  int n_seqs, nq, ring_pages, window, splits, bq, head_chunks;
  float scale;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// 16-byte pieces of `rows` cache rows into a tile of padded shared-memory rows; rows from `nkeys` on become zeros
// (their weights are zero, but what the pool holds there need not be a number).
__device__ __forceinline__ void load_rows(char* dst, const bf16* src, int rows, int nkeys, int tid) {
  constexpr int PPR = D / 8;
  for (int i = tid; i < rows * PPR; i += WARPS * 32) {
    const int j = i / PPR, c = i % PPR;
    char* d = dst + j * ROWB + c * 16;
    if (j < nkeys) cp_async16(smem_addr(d), src + (size_t)j * D + c * 8);
    else *(uint4*)d = make_uint4(0u, 0u, 0u, 0u);
  }
}

__global__ void __launch_bounds__(WARPS * 32)
attention_latent_mma_kernel(LatentAttnArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) char smem[];
  char* Qs = smem;                                   // [ROWS] rows of ROWB bytes
  char* Ks = Qs + Q_BYTES;                           // STAGES tiles of [KT] rows of ROWB bytes
  char* Ps = Ks + STAGES * K_BYTES;                  // [ROWS] rows of P_ROWB bytes
  float* smax = (float*)(Ps + P_BYTES);              // [WARPS][ROWS]
  float* ssum = smax + WARPS * ROWS;                 // [WARPS][ROWS]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int seq = blockIdx.z, chunk = blockIdx.y;
  const int qtile = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
  const int hpb = min(a.nq - chunk * 16, 16);        // query heads of this block
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  const int t0 = qtile * a.bq;
  if (t0 >= q_len) return;
  const int nt = min(a.bq, q_len - t0);
  const int nrows = nt * hpb;
  const int past = a.past[seq];
  const int pos_lo = past + t0, pos_hi = past + t0 + nt - 1;

  int k_lo = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
  k_lo = (k_lo / KT) * KT;
  const int n_tiles = (pos_hi + 1 - k_lo + KT - 1) / KT;
  const int per_split = (n_tiles + a.splits - 1) / a.splits;
  const int tile_begin = split * per_split, tile_end = min(n_tiles, tile_begin + per_split);
  const int n_my = max(tile_end - tile_begin, 0);

  // rows g and g + 8 of the tile: position of the query, -1 for a row without one
  int rpos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    rpos[h] = row < nrows ? past + t0 + row / hpb : -1;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[UPW][2][4];
#pragma unroll
  for (int i = 0; i < UPW; ++i)
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][n][e] = 0.f;

  const int* pages = a.page_ids + a.page_start[seq];
  auto load_tile = [&](int tile, int stage) {
    const int kbase = k_lo + tile * KT;
    const int page = pages[page_slot_of(kbase, PAGE, a.ring_pages)];
    const bf16* src = a.pool + ((size_t)page * PAGE + (kbase % PAGE)) * D;
    load_rows(Ks + stage * K_BYTES, src, KT, min(KT, pos_hi + 1 - kbase), tid);
  };

  if (n_my > 0) {
    // the query rows: row r is token t0 + r / hpb, head chunk * 16 + r % hpb
    constexpr int PPR = D / 8;
    for (int i = tid; i < ROWS * PPR; i += WARPS * 32) {
      const int r = i / PPR, c = i % PPR;
      char* d = Qs + r * ROWB + c * 16;
      if (r < nrows) {
        const int tok = q_begin + t0 + r / hpb, h = chunk * 16 + r % hpb;
        cp_async16(smem_addr(d), a.q + ((size_t)tok * a.nq + h) * D + c * 8);
      } else {
        *(uint4*)d = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    load_tile(tile_begin, 0);
    cp_async_commit();
  }

  // addresses of this lane's rows in the fragment loads
  const uint32_t q_frag = smem_addr(Qs) + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + ((lane >> 4) & 1) * 16;
  const uint32_t p_frag = smem_addr(Ps) + ((lane & 7) + ((lane >> 3) & 1) * 8) * P_ROWB + ((lane >> 4) & 1) * 16;
  const uint32_t k_frag_off = (warp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * ROWB + ((lane >> 3) & 1) * 16;
  const uint32_t v_frag_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + ((lane >> 4) & 1) * 16;
  const float scale2 = a.scale * LOG2E;

  for (int it = 0; it < n_my; ++it) {
    const int tile = tile_begin + it;
    const int stage = STAGES == 2 ? (it & 1) : 0;
    if (STAGES == 2 && it + 1 < n_my) {
      load_tile(tile + 1, (it + 1) & 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kt = smem_addr(Ks) + stage * K_BYTES;

    // scores of this warp's 16 keys for the 16 rows
    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[n][e] = 0.f;
#pragma unroll 4
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t qa[4], b0, b1, b2, b3;
      ldmatrix_x4(q_frag + ks * 32, qa[0], qa[1], qa[2], qa[3]);
      ldmatrix_x4(kt + k_frag_off + ks * 32, b0, b1, b2, b3);
      mma_bf16(sc[0], qa, b0, b1);
      mma_bf16(sc[1], qa, b2, b3);
    }
    const int kbase = k_lo + tile * KT + warp * 16;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kj = kbase + n * 8 + 2 * t + (e & 1), h = e >> 1;
        const bool vis = rpos[h] >= 0 && kj <= rpos[h] && (a.window == 0 || kj > rpos[h] - a.window);
        sc[n][e] = vis ? sc[n][e] * scale2 : -INFINITY;
        mx[h] = fmaxf(mx[h], sc[n][e]);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      if (t == 0) smax[warp * ROWS + g + 8 * h] = mx[h];
    }
    __syncthreads();
    float alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float tm = smax[g + 8 * h];
#pragma unroll
      for (int w = 1; w < WARPS; ++w) tm = fmaxf(tm, smax[w * ROWS + g + 8 * h]);
      const float m_new = fmaxf(m[h], tm);
      alpha[h] = m_new == -INFINITY ? 1.f : exp2f(m[h] - m_new);
      m[h] = m_new;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float p0 = m[h] == -INFINITY ? 0.f : exp2f(sc[n][2 * h] - m[h]);
        const float p1 = m[h] == -INFINITY ? 0.f : exp2f(sc[n][2 * h + 1] - m[h]);
        sum[h] += p0 + p1;
        *(uint32_t*)(Ps + (g + 8 * h) * P_ROWB + (warp * 16 + n * 8 + 2 * t) * 2) = pack_bf16(p0, p1);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
      sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
      if (t == 0) ssum[warp * ROWS + g + 8 * h] = sum[h];
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float ts = ssum[g + 8 * h];
#pragma unroll
      for (int w = 1; w < WARPS; ++w) ts += ssum[w * ROWS + g + 8 * h];
      l[h] = l[h] * alpha[h] + ts;
    }

    // output lanes of this warp: acc = acc * alpha + P V
    uint32_t pa[KT / 16][4];
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) ldmatrix_x4(p_frag + kk * 32, pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3]);
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
      const int u = warp + WARPS * i;
      if (u < UNITS) {
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          acc[i][n][0] *= alpha[0]; acc[i][n][1] *= alpha[0];
          acc[i][n][2] *= alpha[1]; acc[i][n][3] *= alpha[1];
        }
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(kt + v_frag_off + kk * 16 * ROWB + u * 32, b0, b1, b2, b3);
          mma_bf16(acc[i][0], pa[kk], b0, b1);
          mma_bf16(acc[i][1], pa[kk], b2, b3);
        }
      }
    }
    __syncthreads();      // the tile, the weights and the statistics are free again
    if (STAGES == 1 && it + 1 < n_my) {
      load_tile(tile + 1, 0);
      cp_async_commit();
    }
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    if (row >= nrows) continue;
    const int tok = q_begin + t0 + row / hpb, head = chunk * 16 + row % hpb;
    if (a.splits == 1) {
      const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
      bf16* o = a.out + ((size_t)tok * a.nq + head) * DV;
#pragma unroll
      for (int i = 0; i < UPW; ++i) {
        const int u = warp + WARPS * i;
        if (u < UNITS) {
#pragma unroll
          for (int n = 0; n < 2; ++n)
            *(uint32_t*)(o + u * 16 + n * 8 + 2 * t) = pack_bf16(acc[i][n][2 * h] * inv, acc[i][n][2 * h + 1] * inv);
        }
      }
    } else {
      float* o = a.partial + (((size_t)tok * a.nq + head) * a.splits + split) * (DV + 2);
#pragma unroll
      for (int i = 0; i < UPW; ++i) {
        const int u = warp + WARPS * i;
        if (u < UNITS) {
#pragma unroll
          for (int n = 0; n < 2; ++n)
            *(float2*)(o + u * 16 + n * 8 + 2 * t) = make_float2(acc[i][n][2 * h], acc[i][n][2 * h + 1]);
        }
      }
      if (warp == 0 && t == 0) { o[DV] = m[h] == -INFINITY ? -INFINITY : m[h] * LN2; o[DV + 1] = l[h]; }
    }
  }
}

// Merge the partials of one (token, head): out = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s.  The first warp
// turns the splits' maxima and sums into one weight per split (at most 32 splits); then every thread adds up its lanes.
__global__ void attention_latent_combine_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float weight[32];
  const size_t row = blockIdx.x;  // token * nq + head
  const float* p = partial + row * splits * (DV + 2);
  if (threadIdx.x < 32) {
    const int s = threadIdx.x;
    const float ms = s < splits ? p[s * (DV + 2) + DV] : -INFINITY;
    const float ls = s < splits ? p[s * (DV + 2) + DV + 1] : 0.f;
    float M = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float e = ms == -INFINITY ? 0.f : expf(ms - M);
    float denom = e * ls;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    weight[s] = denom > 0.f ? e / denom : 0.f;
  }
  __syncthreads();
  for (int dd = threadIdx.x * 2; dd < DV; dd += blockDim.x * 2) {
    float v0 = 0.f, v1 = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float w = weight[s];
      const float2 x = *(const float2*)(p + s * (DV + 2) + dd);
      // a split without a visible key has weight zero, and zeros as its sums
      v0 = fmaf(w, x.x, v0); v1 = fmaf(w, x.y, v1);
    }
    *(uint32_t*)(out + row * DV + dd) = pack_bf16(v0, v1);
  }
}

extern "C" int odi_attention_latent_mma_dims(int* d, int* dv) { *d = D; *dv = DV; return 0; }

// max_q_len: the longest q_len of the batch (sizes the grid); n_tokens: packed tokens.
extern "C" int odi_attention_latent_mma(const LatentAttnArgs* args, int max_q_len, int n_tokens, int page_size,
                                        cudaStream_t stream) {
  LatentAttnArgs a = *args;
  if (a.n_seqs <= 0 || n_tokens <= 0) return 0;
  if (page_size != PAGE || a.splits < 1 || a.splits > 32 || a.n_seqs > 65535 || a.nq < 1) return ODI_ERR_UNSUPPORTED;
  if (a.splits > 1 && a.partial == nullptr) return ODI_ERR_ARGUMENT;
  const int hpb = a.nq < 16 ? a.nq : 16;
  a.head_chunks = (a.nq + 15) / 16;
  a.bq = ROWS / hpb;
  const int q_tiles = (max_q_len + a.bq - 1) / a.bq;
  dim3 grid(q_tiles * a.splits, a.head_chunks, a.n_seqs);
  if (grid.y > 65535) return ODI_ERR_UNSUPPORTED;
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(attention_latent_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  odi_rc = launch_pdl(attention_latent_mma_kernel, grid, dim3(WARPS * 32), (size_t)SMEM_BYTES, stream, a);
  const int rc = launch_status();
  if (rc != 0 || a.splits == 1) return rc;
  const int threads = DV >= 512 ? 256 : (DV >= 256 ? 128 : (DV >= 128 ? 64 : 32));
  odi_rc = launch_pdl(attention_latent_combine_kernel, dim3(n_tokens * a.nq), dim3(threads), 0, stream,
                      (const float*)a.partial, a.out, a.splits);
  return launch_status();
}
