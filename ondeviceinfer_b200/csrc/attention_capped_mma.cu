// bf16 causal grouped-query attention with squashed scores, a window and a value width of its own, over the
// paged cache (a ring of pages per sequence for a windowed layer), on the tensor cores: mma.sync m16n8k16 with
// fp32 accumulation, fp32 scores, cap and running-maximum softmax.
//
// A block of 4 warps owns 64 consecutive query tokens of one query head of one sequence (16 rows per warp) and
// walks the key tiles of 64 positions from the first one that its oldest query still sees to the diagonal; it
// works for any q_len >= 1 on top of any cached length, so prompts, their portions and single tokens all fit
// (single tokens go to the second kernel of this file, which cuts the keys among blocks).
//
//   score = q . k * scale;  with softcap c > 0: score <- c tanh(score / c);  with sink = 1 the softmax has one more
//   term, of score 0 and without a value: p_j = e^(s_j) / (1 + sum_k e^(s_k));
//   key j is visible to the query at position p iff j <= p and (window == 0 or j > p - window or j < keep): with
//   keep > 0 a windowed layer goes on seeing the first `keep` positions of its sequence; their tiles come first in
//   a block's walk, then the tiles of the window.
//
// Key and value tiles (64 positions x D resp. DV bf16, contiguous in a page) are copied with cp.async, double
// buffered, one block barrier per tile, into rows padded by 16 bytes so that ldmatrix reads are free of bank
// conflicts.  Compile with -DODI_HEAD_DIM=<D> -DODI_VALUE_DIM=<DV>, multiples of 16 up to 256.
#include "common.cuh"

#ifndef ODI_HEAD_DIM
#error "compile with -DODI_HEAD_DIM=<key width> -DODI_VALUE_DIM=<value width>"
#endif
#ifndef ODI_VALUE_DIM
#define ODI_VALUE_DIM ODI_HEAD_DIM
#endif
#define D ODI_HEAD_DIM
#define DV ODI_VALUE_DIM
#if (D % 16) != 0 || D > 256 || (DV % 16) != 0 || DV > 256
#error "key and value widths must be multiples of 16, at most 256"
#endif

#define KT 64                       // keys per tile = positions per page
#define ROWB_K (2 * D + 16)         // bytes per shared-memory row of a key tile
#define ROWB_V (2 * DV + 16)
#define K_BYTES (KT * ROWB_K)
#define V_BYTES (KT * ROWB_V)
#define KSTEPS (D / 16)
#define DVTILES (DV / 8)
#define LOG2E 1.4426950408889634f
#define WARPS 4
#define STAGES 2

struct CappedAttnArgs {
  const bf16* q;          // [n_tokens, nq, D]
  const bf16* k_pool;     // [pages, nkv, 64, D]
  const bf16* v_pool;     // [pages, nkv, 64, DV]
  bf16* out;              // [n_tokens, nq * DV]
  const int* cu_q;
  const int* past;
  const int* page_start;
  const int* page_ids;
  int n_seqs, nq, nkv, ring_pages, window;
  float scale, softcap;
  int sink;               // 1: the softmax has one more term, of score 0 and without a value
  int keep;               // > 0 with a window: keys 0..keep-1 stay visible beyond the window
};

// 1 / (l + 2^-m) for row sums l taken relative to the maximum m (log2 domain): the denominator with the sink's
// term, without overflow; zero for a row that saw no key.
__device__ __forceinline__ float sink_inverse_log2(float m, float l) {
  if (m == -INFINITY) return 0.f;
  if (m >= 0.f) return 1.f / (l + exp2f(-m));
  const float e = exp2f(m);
  return e / fmaf(l, e, 1.f);
}

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

// One page tile (64 rows of W bf16, contiguous in global memory) into rows of ROWB bytes.
template <int W, int ROWB>
__device__ __forceinline__ void load_tile(uint8_t* dst, const bf16* src, int tid) {
  constexpr int CHUNKS = W / 8;    // 16-byte chunks per row
  const uint32_t base = smem_addr(dst);
  for (int i = tid; i < KT * CHUNKS; i += WARPS * 32) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    cp_async16(base + r * ROWB + c * 16, src + (size_t)r * W + c * 8);
  }
}

// A score times scale, squashed, in the log2 domain.  tanh(x) = 1 - 2 / (e^(2x) + 1): its absolute error stays at
// a few 1e-7 over the whole range (e^(2x) overflows to +inf and gives 1, underflows to 0 and gives -1).
__device__ __forceinline__ float shape_score(float s, float scale, float cap, float two_over_cap) {
  s *= scale;
  if (cap > 0.f) s = cap * (1.f - __fdividef(2.f, __expf(s * two_over_cap) + 1.f));
  return s * LOG2E;
}

__global__ void __launch_bounds__(WARPS * 32)
attention_capped_kernel(CappedAttnArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // heads along x, sequences along y, query tiles along z from the last (the most keys) to the first
  const int seq = blockIdx.y, head = blockIdx.x, hk = head / (a.nq / a.nkv);
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  const int t0 = (gridDim.z - 1 - blockIdx.z) * 64;
  if (t0 >= q_len) return;
  const int past = a.past[seq];
  const int nt = min(64, q_len - t0);
  const int first_key = a.window > 0 ? max(0, past + t0 - a.window + 1) : 0;     // the oldest key any row sees
  const int tile_lo = first_key / KT, tile_hi = (past + t0 + nt - 1) / KT;       // inclusive
  // the walk: the tiles of kept first keys in front of the window's first tile, then tile_lo..tile_hi
  const int keep_tiles = a.window > 0 && a.keep > 0 ? min((a.keep + KT - 1) / KT, tile_lo) : 0;
  const int n_walk = keep_tiles + tile_hi - tile_lo + 1;
  auto tile_of = [&](int w) { return w < keep_tiles ? w : tile_lo + (w - keep_tiles); };
  const int* pages = a.page_ids + a.page_start[seq];

  // this warp's rows: tokens t0 + warp*16 + {lane/4, lane/4 + 8}
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const bf16* q_lo = r_lo < nt ? a.q + ((size_t)(q_begin + t0 + r_lo) * a.nq + head) * D : nullptr;
  const bf16* q_hi = r_hi < nt ? a.q + ((size_t)(q_begin + t0 + r_hi) * a.nq + head) * D : nullptr;
  uint32_t qf[KSTEPS][4];
  {
    const int c = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      qf[ks][0] = q_lo ? *(const uint32_t*)(q_lo + ks * 16 + c) : 0u;
      qf[ks][1] = q_hi ? *(const uint32_t*)(q_hi + ks * 16 + c) : 0u;
      qf[ks][2] = q_lo ? *(const uint32_t*)(q_lo + ks * 16 + 8 + c) : 0u;
      qf[ks][3] = q_hi ? *(const uint32_t*)(q_hi + ks * 16 + 8 + c) : 0u;
    }
  }
  const int pos_lo = past + t0 + r_lo, pos_hi = past + t0 + r_hi;
  // the oldest key of each row: everything from 0 without a window
  const int old_lo = a.window > 0 ? pos_lo - a.window + 1 : 0, old_hi = a.window > 0 ? pos_hi - a.window + 1 : 0;

  float o[DVTILES][4];
#pragma unroll
  for (int i = 0; i < DVTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const float two_over_cap = a.softcap > 0.f ? 2.f / a.softcap : 0.f;

  auto issue = [&](int w) {
    uint8_t* st = smem + (size_t)(w % STAGES) * (K_BYTES + V_BYTES);
    const int page = pages[page_slot_of_page(tile_of(w), a.ring_pages)];
    const size_t row0 = ((size_t)page * a.nkv + hk) * KT;
    load_tile<D, ROWB_K>(st, a.k_pool + row0 * D, tid);
    load_tile<DV, ROWB_V>(st + K_BYTES, a.v_pool + row0 * DV, tid);
    cp_async_commit();
  };
  issue(0);
  for (int w = 0; w < n_walk; ++w) {
    if (w + 1 < n_walk) { issue(w + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint8_t* st = smem + (size_t)(w % STAGES) * (K_BYTES + V_BYTES);
    const uint32_t k_smem = smem_addr(st), v_smem = k_smem + K_BYTES;
    const int kbase = tile_of(w) * KT;
    // a warp whose rows all lie before this tile, or all see only later keys, has nothing to add
    const int warp_first = past + t0 + warp * 16, warp_last = warp_first + 15;
    const bool active = kbase <= warp_last && (a.window == 0 || kbase + KT - 1 > warp_first - a.window || kbase < a.keep);
    if (active) {
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {     // pairs of 8-key tiles
          // matrices: (keys np*16 + 0..7, d ks*16 + 0..7), (same keys, d + 8), (keys + 8, d), (keys + 8, d + 8)
          const int m = lane >> 3, r = lane & 7;
          const int key = np * 16 + (m >> 1) * 8 + r, dd = ks * 16 + (m & 1) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(k_smem + key * ROWB_K + dd * 2, b0, b1, b2, b3);
          mma_bf16(s[np * 2], qf[ks], b0, b1);
          mma_bf16(s[np * 2 + 1], qf[ks], b2, b3);
        }
      }
      // scale, cap, mask, running maximum (log2 domain)
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int kj = kbase + i * 8 + (lane & 3) * 2;
        s[i][0] = (kj <= pos_lo && (kj >= old_lo || kj < a.keep)) ? shape_score(s[i][0], a.scale, a.softcap, two_over_cap) : -INFINITY;
        s[i][1] = (kj + 1 <= pos_lo && (kj + 1 >= old_lo || kj + 1 < a.keep)) ? shape_score(s[i][1], a.scale, a.softcap, two_over_cap) : -INFINITY;
        s[i][2] = (kj <= pos_hi && (kj >= old_hi || kj < a.keep)) ? shape_score(s[i][2], a.scale, a.softcap, two_over_cap) : -INFINITY;
        s[i][3] = (kj + 1 <= pos_hi && (kj + 1 >= old_hi || kj + 1 < a.keep)) ? shape_score(s[i][3], a.scale, a.softcap, two_over_cap) : -INFINITY;
        mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      // rows with nothing visible yet keep a zero accumulator; avoid (-inf) - (-inf)
      const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float al_lo = exp2f(m_lo - ref_lo), al_hi = exp2f(m_hi - ref_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
      uint32_t pf[4][4];                  // P as A fragments for the 4 key steps of 16
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p0 = exp2f(s[i][0] - ref_lo), p1 = exp2f(s[i][1] - ref_lo);
        const float p2 = exp2f(s[i][2] - ref_hi), p3 = exp2f(s[i][3] - ref_hi);
        sum_lo += p0 + p1; sum_hi += p2 + p3;
        pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
        pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      l_lo = l_lo * al_lo + sum_lo; l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DVTILES; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {      // 16 keys per step
#pragma unroll
        for (int dp = 0; dp < DVTILES / 2; ++dp) {
          // matrices: (keys kk*16 + 0..7, d dp*16 + 0..7), (keys + 8, same d), (keys, d + 8), (keys + 8, d + 8)
          const int m = lane >> 3, r = lane & 7;
          const int key = kk * 16 + (m & 1) * 8 + r, dd = dp * 16 + (m >> 1) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(v_smem + key * ROWB_V + dd * 2, b0, b1, b2, b3);
          mma_bf16(o[dp * 2], pf[kk], b0, b1);
          mma_bf16(o[dp * 2 + 1], pf[kk], b2, b3);
        }
      }
    }
    __syncthreads();    // the stage may be overwritten by the load after next
  }
  // the row sums live spread over the 4 lanes of a quad
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  if (a.sink) { inv_lo = sink_inverse_log2(m_lo, l_lo); inv_hi = sink_inverse_log2(m_hi, l_hi); }
  const int c = (lane & 3) * 2;
  if (r_lo < nt) {
    bf16* dst = a.out + ((size_t)(q_begin + t0 + r_lo) * a.nq + head) * DV;
#pragma unroll
    for (int i = 0; i < DVTILES; ++i) *(uint32_t*)(dst + i * 8 + c) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
  }
  if (r_hi < nt) {
    bf16* dst = a.out + ((size_t)(q_begin + t0 + r_hi) * a.nq + head) * DV;
#pragma unroll
    for (int i = 0; i < DVTILES; ++i) *(uint32_t*)(dst + i * 8 + c) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
  }
}

// ------------------------------------------------------------------------------ single tokens
//
// One query token per sequence.  A block owns one (sequence, kv head, split of the visible keys); the rows of its
// MMA are the query heads that share the kv head (up to 16 per block); its 4 warps take 16 keys each of every
// 64-key tile and merge their partial results in shared memory.  With several splits the block writes its merged
// (acc[DV], max, sum) to global memory (a split without keys writes max = -inf) and the combine kernel adds the
// splits of a (token, head) in order.

struct CappedDecodeArgs {
  CappedAttnArgs base;
  float* partial;         // [n_tokens, nq, splits, DV + 2]
  int splits, head_chunks;
};

__global__ void __launch_bounds__(WARPS * 32)
attention_capped_decode_kernel(CappedDecodeArgs da) {
  pdl_launch_dependents();
  pdl_wait();
  const CappedAttnArgs& a = da.base;
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, seq = blockIdx.z;
  const int hk = blockIdx.y / da.head_chunks, chunk = blockIdx.y % da.head_chunks;
  const int g = a.nq / a.nkv;
  const int heads_here = min(16, g - chunk * 16);
  const int head0 = hk * g + chunk * 16;
  const int tok = a.cu_q[seq];
  const int pos = a.past[seq];                     // the query's position
  const int first_key = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  // the walk over all splits: the tiles of kept first keys in front of the window's first tile, then the window's
  const int tile_lo = first_key / KT;
  const int keep_tiles = a.window > 0 && a.keep > 0 ? min((a.keep + KT - 1) / KT, tile_lo) : 0;
  const int n_tiles = keep_tiles + pos / KT + 1 - tile_lo;
  auto tile_of = [&](int w) { return w < keep_tiles ? w : tile_lo + (w - keep_tiles); };
  const int per_split = (n_tiles + da.splits - 1) / da.splits;
  const int tile_begin = split * per_split, tile_end = min(n_tiles, tile_begin + per_split);     // places in the walk
  const int* pages = a.page_ids + a.page_start[seq];
  constexpr int RS = DV + 2;
  if (tile_begin >= tile_end) {
    // nothing to see: say so to the combine kernel (only reached with several splits)
    for (int row = warp; row < heads_here; row += WARPS)
      if (lane == 0) {
        float* dst = da.partial + (((size_t)tok * a.nq + head0 + row) * da.splits + split) * RS;
        dst[DV] = -INFINITY; dst[DV + 1] = 0.f;
      }
    return;
  }

  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  const bf16* q_lo = r_lo < heads_here ? a.q + ((size_t)tok * a.nq + head0 + r_lo) * D : nullptr;
  const bf16* q_hi = r_hi < heads_here ? a.q + ((size_t)tok * a.nq + head0 + r_hi) * D : nullptr;
  uint32_t qf[KSTEPS][4];
  {
    const int c = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      qf[ks][0] = q_lo ? *(const uint32_t*)(q_lo + ks * 16 + c) : 0u;
      qf[ks][1] = q_hi ? *(const uint32_t*)(q_hi + ks * 16 + c) : 0u;
      qf[ks][2] = q_lo ? *(const uint32_t*)(q_lo + ks * 16 + 8 + c) : 0u;
      qf[ks][3] = q_hi ? *(const uint32_t*)(q_hi + ks * 16 + 8 + c) : 0u;
    }
  }
  float o[DVTILES][4];
#pragma unroll
  for (int i = 0; i < DVTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const float two_over_cap = a.softcap > 0.f ? 2.f / a.softcap : 0.f;

  auto issue = [&](int tile) {
    uint8_t* st = smem + (size_t)((tile - tile_begin) % STAGES) * (K_BYTES + V_BYTES);
    const int page = pages[page_slot_of_page(tile_of(tile), a.ring_pages)];
    const size_t row0 = ((size_t)page * a.nkv + hk) * KT;
    load_tile<D, ROWB_K>(st, a.k_pool + row0 * D, tid);
    load_tile<DV, ROWB_V>(st + K_BYTES, a.v_pool + row0 * DV, tid);
    cp_async_commit();
  };
  issue(tile_begin);
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    if (tile + 1 < tile_end) { issue(tile + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint8_t* st = smem + (size_t)((tile - tile_begin) % STAGES) * (K_BYTES + V_BYTES);
    const uint32_t k_smem = smem_addr(st), v_smem = k_smem + K_BYTES;
    const int kbase = tile_of(tile) * KT + warp * 16;        // this warp's 16 keys
    if (kbase <= pos && (kbase + 15 >= first_key || kbase < a.keep)) {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int m = lane >> 3, r = lane & 7;
        const int key = warp * 16 + (m >> 1) * 8 + r, dd = ks * 16 + (m & 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(k_smem + key * ROWB_K + dd * 2, b0, b1, b2, b3);
        mma_bf16(s[0], qf[ks], b0, b1);
        mma_bf16(s[1], qf[ks], b2, b3);
      }
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int kj = kbase + i * 8 + (lane & 3) * 2;
        const bool v0 = kj <= pos && (kj >= first_key || kj < a.keep), v1 = kj + 1 <= pos && (kj + 1 >= first_key || kj + 1 < a.keep);
        s[i][0] = v0 ? shape_score(s[i][0], a.scale, a.softcap, two_over_cap) : -INFINITY;
        s[i][1] = v1 ? shape_score(s[i][1], a.scale, a.softcap, two_over_cap) : -INFINITY;
        s[i][2] = v0 ? shape_score(s[i][2], a.scale, a.softcap, two_over_cap) : -INFINITY;
        s[i][3] = v1 ? shape_score(s[i][3], a.scale, a.softcap, two_over_cap) : -INFINITY;
        mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);   // finite: one of the 16 keys is visible
      const float al_lo = exp2f(m_lo - mn_lo), al_hi = exp2f(m_hi - mn_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      uint32_t pf[4];
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float p0 = exp2f(s[i][0] - mn_lo), p1 = exp2f(s[i][1] - mn_lo);
        const float p2 = exp2f(s[i][2] - mn_hi), p3 = exp2f(s[i][3] - mn_hi);
        sum_lo += p0 + p1; sum_hi += p2 + p3;
        pf[i * 2] = pack_bf16(p0, p1);
        pf[i * 2 + 1] = pack_bf16(p2, p3);
      }
      l_lo = l_lo * al_lo + sum_lo; l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DVTILES; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
#pragma unroll
      for (int dp = 0; dp < DVTILES / 2; ++dp) {
        const int m = lane >> 3, r = lane & 7;
        const int key = warp * 16 + (m & 1) * 8 + r, dd = dp * 16 + (m >> 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(v_smem + key * ROWB_V + dd * 2, b0, b1, b2, b3);
        mma_bf16(o[dp * 2], pf, b0, b1);
        mma_bf16(o[dp * 2 + 1], pf, b2, b3);
      }
    }
    __syncthreads();
  }
  // merge the four warps (each saw a quarter of the keys): [warp][row][DV + 2] floats over the free tiles
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  float* mg = (float*)smem;
  {
    const int c = (lane & 3) * 2;
    float* lo = mg + ((size_t)warp * 16 + r_lo) * RS;
    float* hi = mg + ((size_t)warp * 16 + r_hi) * RS;
#pragma unroll
    for (int i = 0; i < DVTILES; ++i) {
      lo[i * 8 + c] = o[i][0]; lo[i * 8 + c + 1] = o[i][1];
      hi[i * 8 + c] = o[i][2]; hi[i * 8 + c + 1] = o[i][3];
    }
    if ((lane & 3) == 0) { lo[DV] = m_lo; lo[DV + 1] = l_lo; hi[DV] = m_hi; hi[DV + 1] = l_hi; }
  }
  __syncthreads();
  for (int row = warp; row < heads_here; row += WARPS) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, mg[((size_t)w * 16 + row) * RS + DV]);
    float wgt[WARPS], L = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = mg[((size_t)w * 16 + row) * RS + DV];
      wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += wgt[w] * mg[((size_t)w * 16 + row) * RS + DV + 1];
    }
    const int head = head0 + row;
    if (da.splits == 1) {
      float inv = L > 0.f ? 1.f / L : 0.f;
      if (a.sink) inv = sink_inverse_log2(M, L);
      bf16* dst = a.out + ((size_t)tok * a.nq + head) * DV;
      for (int dd = lane; dd < DV; dd += 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += wgt[w] * mg[((size_t)w * 16 + row) * RS + dd];
        dst[dd] = __float2bfloat16_rn(v * inv);
      }
    } else {
      // partial in the natural-log domain of the combine kernel: max * ln 2
      float* dst = da.partial + (((size_t)tok * a.nq + head) * da.splits + split) * RS;
      for (int dd = lane; dd < DV; dd += 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += wgt[w] * mg[((size_t)w * 16 + row) * RS + dd];
        dst[dd] = v;
      }
      if (lane == 0) { dst[DV] = M == -INFINITY ? -INFINITY : M * 0.6931471805599453f; dst[DV + 1] = L; }
    }
  }
}

// Merge the partials of one (token, head): out = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s, splits in order.
__global__ void attention_capped_combine_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int splits,
                                                int sink) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int RS = DV + 2;
  const size_t row = blockIdx.x;  // token * nq + head
  const float* p = partial + row * splits * RS;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, p[s * RS + DV]);
  float denom = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = p[s * RS + DV];
    if (ms != -INFINITY) denom += expf(ms - M) * p[s * RS + DV + 1];
  }
  float inv = denom > 0.f ? 1.f / denom : 0.f;
  if (sink) inv = sink_inverse_log2(M * LOG2E, denom);      // the partials' maxima are natural logarithms
  for (int dd = threadIdx.x; dd < DV; dd += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = p[s * RS + DV];
      if (ms != -INFINITY) v += expf(ms - M) * p[s * RS + dd];
    }
    out[row * DV + dd] = __float2bfloat16_rn(v * inv);
  }
}

// One token per sequence; `partial` holds n_seqs * nq * splits * (DV + 2) floats when splits > 1.
extern "C" int odi_attention_capped_decode(const CappedAttnArgs* args, float* partial, int splits, cudaStream_t stream) {
  CappedDecodeArgs da;
  da.base = *args;
  const CappedAttnArgs& a = da.base;
  if (a.n_seqs <= 0) return 0;
  if (a.nkv <= 0 || a.nq % a.nkv != 0 || a.n_seqs > 65535 || a.window < 0 || a.ring_pages < 0 || a.keep < 0 || splits < 1) return ODI_ERR_UNSUPPORTED;
  if (((uintptr_t)a.q | (uintptr_t)a.k_pool | (uintptr_t)a.v_pool | (uintptr_t)a.out) % 16 != 0) return ODI_ERR_UNSUPPORTED;
  if (splits > 1 && partial == nullptr) return ODI_ERR_ARGUMENT;
  da.partial = partial;
  da.splits = splits;
  da.head_chunks = (a.nq / a.nkv + 15) / 16;
  const dim3 grid(splits, a.nkv * da.head_chunks, a.n_seqs);
  if (grid.y > 65535) return ODI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)STAGES * (K_BYTES + V_BYTES);
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(attention_capped_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  odi_rc = launch_pdl(attention_capped_decode_kernel, grid, dim3(WARPS * 32), smem, stream, da);
  int rc = launch_status();
  if (rc != 0 || splits == 1) return rc;
  const int rows = a.n_seqs * a.nq;
  const int threads = DV >= 128 ? 128 : (DV >= 64 ? 64 : 32);
  odi_rc = launch_pdl(attention_capped_combine_kernel, dim3(rows), dim3(threads), 0, stream, (const float*)partial, a.out, splits, a.sink);
  return launch_status();
}

extern "C" int odi_attention_capped_dims(int* d, int* dv) { *d = D; *dv = DV; return 0; }

// max_q_len: the longest q_len of the batch (sizes the grid).
extern "C" int odi_attention_capped(const CappedAttnArgs* args, int max_q_len, cudaStream_t stream) {
  const CappedAttnArgs a = *args;
  if (a.n_seqs <= 0 || max_q_len <= 0) return 0;
  if (a.nkv <= 0 || a.nq % a.nkv != 0 || a.n_seqs > 65535 || a.window < 0 || a.ring_pages < 0 || a.keep < 0) return ODI_ERR_UNSUPPORTED;
  if (((uintptr_t)a.q | (uintptr_t)a.k_pool | (uintptr_t)a.v_pool | (uintptr_t)a.out) % 16 != 0) return ODI_ERR_UNSUPPORTED;
  const int q_tiles = (max_q_len + 63) / 64;
  if (q_tiles > 65535) return ODI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)STAGES * (K_BYTES + V_BYTES);
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(attention_capped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  odi_rc = launch_pdl(attention_capped_kernel, dim3(a.nq, a.n_seqs, q_tiles), dim3(WARPS * 32), smem, stream, a);
  return launch_status();
}
