// Grouped matrix product on the CUDA cores: many small products C_g = A_g W_g^T in one launch, each group with
// a weight matrix of its own.  fp32 accumulation over k = 0..K-1 in that order for every output element,
// whatever else is in the launch, for both element types (T = float: the true 32-bit path; T = bf16).
//
// Two ways to say which rows belong to which group:
//  * dense (tile table null): every group has the same M rows; group g reads columns [g * a_group_off, +K) of
//    A's rows 0..M-1 and writes columns [g * c_group_off, +N) of C's rows (a product per head);
//  * by table (routed experts): tile t covers `tile_rows[t]` rows from `tile_row0[t]` on, in an order sorted
//    by group, all of group `tile_group[t]`; `n_tiles[0]` tiles exist (blocks beyond it leave).  Row i of that
//    order reads row `row_index[i] / index_div` of A (row i itself if row_index is null) and writes row i of C.
//
// Epilogues: 0 store as T, 1 store as fp32, 2 gated and clamped (W_g holds N gate rows then N up rows;
// g = min(gate, limit), u = clamp(up, -limit, limit), C = g * sigmoid(alpha * g) * (u + 1) as T), 3 the exact
// (erf) GELU of the sum as T, 4 its tanh form, 5 the square of max(sum, 0) as T.
//
// Tile: TM rows x 64 features per block of 256 threads, K in slices of 16 or 32 through shared memory (fp32).
// TM = 64 (4 x 4 outputs a thread) or 16 (1 x 4), chosen by the caller from the rows a group has; for groups
// of a few rows there is a form that streams the weights through registers only (grouped_gemv_kernel).
#include "common.cuh"
#include <algorithm>
#include <cstring>
#include <type_traits>

#define TN 64

__device__ __forceinline__ float grouped_act(float z, int epi) {
  if (epi == 3) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (epi == 4) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  if (epi == 5) { const float r = fmaxf(z, 0.f); return r * r; }
  return z;
}

struct GroupedArgs {
  const void* A;
  const void* W;
  void* C;
  const int* row_index;
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* n_tiles;
  long long a_group_off, w_group_stride, c_group_off;
  int lda, ldw, ldc, M, N, K, groups, index_div, epi;
  float limit, alpha;
};

// Eight consecutive elements of a row as floats (16-byte loads; the caller has checked the alignment).
template <typename T> __device__ __forceinline__ void load8(const T* p, float* out);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* out) {
  const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* out) {
  const uint4 raw = *(const uint4*)p;
  const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}

// A k-major tile in shared memory, [TK][STR] floats with 8 more floats after every 8 k: the four 8-element
// pieces of a row's 32 k land in different banks when one warp stores them.
#define SIDX(k, i, STR) ((k) * (STR) + ((k) >> 3) * 8 + (i))

// VEC: K, the row strides and the group offsets are multiples of 8 elements and the bases 16-byte aligned:
// slices of 32 k, one 8-element piece per thread and tile; else slices of 16 k, element by element.
template <typename T, int TM, bool GATED, bool VEC>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(GroupedArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int RPT = TM / 16;
  constexpr int TK = VEC ? 32 : 16;
  constexpr int ASTR = TM + 4, WSTR = TN + 4;
  __shared__ __align__(16) float As[TK * ASTR + (TK / 8) * 8];
  __shared__ __align__(16) float Ws[GATED ? 2 : 1][TK * WSTR + (TK / 8) * 8];
  __shared__ int arow[TM];
  const int tid = threadIdx.x;
  int group, row0, rows;
  if (a.tile_group != nullptr) {
    const int t = blockIdx.x;
    if (t >= a.n_tiles[0]) return;
    group = a.tile_group[t]; row0 = a.tile_row0[t]; rows = a.tile_rows[t];
  } else {
    group = blockIdx.z; row0 = blockIdx.x * TM; rows = min(TM, a.M - row0);
  }
  const int n0 = blockIdx.y * TN;
  if (tid < TM) {
    int r = -1;
    if (tid < rows) r = a.row_index != nullptr ? a.row_index[row0 + tid] / a.index_div : row0 + tid;
    arow[tid] = r;
  }
  __syncthreads();
  const T* A = (const T*)a.A + (a.tile_group != nullptr ? 0 : (size_t)group * a.a_group_off);
  const T* W = (const T*)a.W + (size_t)group * a.w_group_stride;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[GATED ? 2 : 1][RPT][4] = {};

  // VEC: the pieces of the next slice are requested while the current one is multiplied
  float va[8], vw[GATED ? 2 : 1][8];
  const int piece = tid & 3, vrow = tid >> 2;
  auto fetch = [&](int k0) {
    const int k = k0 + piece * 8;
    const int src = tid < TM * 4 ? arow[vrow] : -1;
    if (src >= 0 && k < a.K) load8<T>(A + (size_t)src * a.lda + k, va);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) va[i] = 0.f;
    }
    const bool in = n0 + vrow < a.N && k < a.K;
#pragma unroll
    for (int s = 0; s < (GATED ? 2 : 1); ++s) {
      if (in) load8<T>(W + (size_t)(s * a.N + n0 + vrow) * a.ldw + k, vw[s]);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) vw[s][i] = 0.f;
      }
    }
  };
  if (VEC) fetch(0);

  for (int k0 = 0; k0 < a.K; k0 += TK) {
    __syncthreads();
    if (VEC) {
      if (tid < TM * 4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) As[SIDX(piece * 8 + i, vrow, ASTR)] = va[i];
      }
#pragma unroll
      for (int s = 0; s < (GATED ? 2 : 1); ++s) {
#pragma unroll
        for (int i = 0; i < 8; ++i) Ws[s][SIDX(piece * 8 + i, vrow, WSTR)] = vw[s][i];
      }
      if (k0 + TK < a.K) fetch(k0 + TK);
    } else {
      for (int i = tid; i < TM * TK; i += 256) {
        const int r = i / TK, k = i % TK;
        const int src = arow[r];
        As[SIDX(k, r, ASTR)] = (src >= 0 && k0 + k < a.K) ? to_f<T>(A[(size_t)src * a.lda + k0 + k]) : 0.f;
      }
      for (int i = tid; i < TN * TK; i += 256) {
        const int n = i / TK, k = i % TK;
        const bool in = n0 + n < a.N && k0 + k < a.K;
        Ws[0][SIDX(k, n, WSTR)] = in ? to_f<T>(W[(size_t)(n0 + n) * a.ldw + k0 + k]) : 0.f;
        if (GATED) Ws[1][SIDX(k, n, WSTR)] = in ? to_f<T>(W[(size_t)(a.N + n0 + n) * a.ldw + k0 + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float ar[RPT];
#pragma unroll
      for (int i = 0; i < RPT; ++i) ar[i] = As[SIDX(k, ty * RPT + i, ASTR)];
#pragma unroll
      for (int s = 0; s < (GATED ? 2 : 1); ++s) {
        const float4 wv = *(const float4*)&Ws[s][SIDX(k, tx * 4, WSTR)];
        const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < RPT; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[s][i][j] = fmaf(ar[i], wr[j], acc[s][i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = ty * RPT + i;
    if (r >= rows) continue;
    const size_t crow = (size_t)(row0 + r) * a.ldc + (a.tile_group != nullptr ? 0 : (size_t)group * a.c_group_off);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      if (GATED) {
        const float g = fminf(acc[0][i][j], a.limit);
        const float u = fminf(fmaxf(acc[GATED ? 1 : 0][i][j], -a.limit), a.limit);
        ((T*)a.C)[crow + n] = from_f<T>(g / (1.f + expf(-a.alpha * g)) * (u + 1.f));
      } else if (a.epi == 1) {
        ((float*)a.C)[crow + n] = acc[0][i][j];
      } else {
        ((T*)a.C)[crow + n] = from_f<T>(grouped_act(acc[0][i][j], a.epi));
      }
    }
  }
}

// Few rows per group (single-token steps): no tile of the weights in shared memory.  A block takes up to 4 rows
// of one group and 64 features (32 in the gated form); the rows wait in shared memory as floats, each of the 8 warps takes 8 weight
// rows (for the gated form 4 features: their gate and up rows), a lane reads 8 consecutive k of each weight row
// per step (16-byte loads, eight in flight) and keeps one sum per weight row and input row; sums are reduced over
// the lanes at the end (a fixed tree: the result of a row does not depend on the other rows of the launch).
// Needs what VEC needs.
#define GV_ROWS 4
template <typename T, bool GATED>
__global__ void __launch_bounds__(256, 2)
grouped_gemv_kernel(GroupedArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xs[];       // [GV_ROWS][K]
  __shared__ int arow[GV_ROWS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int group, row0, rows;
  if (a.tile_group != nullptr) {
    const int t = blockIdx.x;
    if (t >= a.n_tiles[0]) return;
    group = a.tile_group[t]; row0 = a.tile_row0[t]; rows = a.tile_rows[t];
  } else {
    group = blockIdx.z; row0 = blockIdx.x * GV_ROWS; rows = min(GV_ROWS, a.M - row0);
  }
  if (tid < GV_ROWS) {
    int r = -1;
    if (tid < rows) r = a.row_index != nullptr ? a.row_index[row0 + tid] / a.index_div : row0 + tid;
    arow[tid] = r;
  }
  __syncthreads();
  const T* A = (const T*)a.A + (a.tile_group != nullptr ? 0 : (size_t)group * a.a_group_off);
  const T* W = (const T*)a.W + (size_t)group * a.w_group_stride;
  for (int i = tid * 8; i < GV_ROWS * a.K; i += 256 * 8) {
    const int r = i / a.K, k = i % a.K;
    float v[8];
    if (arow[r] >= 0) load8<T>(A + (size_t)arow[r] * a.lda + k, v);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) xs[i + j] = v[j];
  }
  __syncthreads();
  // weight row j of this warp: plain form feature n0 + warp * 8 + j; gated form feature n0 + warp * 4 + j / 2,
  // its gate row (j even) or up row (j odd)
  const int n0 = blockIdx.y * (GATED ? 32 : 64);      // 8 warps x 8 weight rows: 64 features, or 32 gated ones
  const T* wrow[8];
  bool wlive[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int n = GATED ? n0 + warp * 4 + (j >> 1) : n0 + warp * 8 + j;
    wlive[j] = n < a.N;
    wrow[j] = W + (size_t)((GATED && (j & 1)) ? a.N + n : n) * a.ldw;
  }
  float acc[8][GV_ROWS] = {};
  for (int k = lane * 8; k < a.K; k += 256) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {       // four weight rows at a time: fewer registers, two blocks per SM
      float w[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (wlive[half * 4 + j]) load8<T>(wrow[half * 4 + j] + k, w[j]);
        else {
#pragma unroll
          for (int e = 0; e < 8; ++e) w[j][e] = 0.f;
        }
      }
#pragma unroll
      for (int r = 0; r < GV_ROWS; ++r) {
        const float4 x0 = *(const float4*)&xs[r * a.K + k], x1 = *(const float4*)&xs[r * a.K + k + 4];
        const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[half * 4 + j][r] = fmaf(w[j][e], x[e], acc[half * 4 + j][r]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int r = 0; r < GV_ROWS; ++r) acc[j][r] = warp_sum(acc[j][r]);
  if (lane != 0) return;
#pragma unroll
  for (int r = 0; r < GV_ROWS; ++r) {
    if (r >= rows) continue;
    const size_t crow = (size_t)(row0 + r) * a.ldc + (a.tile_group != nullptr ? 0 : (size_t)group * a.c_group_off);
    if (GATED) {
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int n = n0 + warp * 4 + f;
        if (n >= a.N) continue;
        const float g = fminf(acc[2 * f][r], a.limit);
        const float u = fminf(fmaxf(acc[2 * f + 1][r], -a.limit), a.limit);
        ((T*)a.C)[crow + n] = from_f<T>(g / (1.f + expf(-a.alpha * g)) * (u + 1.f));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = n0 + warp * 8 + j;
        if (n >= a.N) continue;
        if (a.epi == 1) ((float*)a.C)[crow + n] = acc[j][r];
        else ((T*)a.C)[crow + n] = from_f<T>(grouped_act(acc[j][r], a.epi));
      }
    }
  }
}

// bf16 with the weights streamed through shared memory by cp.async: every lane keeps several requests of 16 bytes per
// weight row in flight and later reads exactly the bytes it asked for, so the ring needs no barrier, and the stream
// is decoupled from the arithmetic: far more bytes on their way per SM than the registers of the form above can hold.
#define GS_CHUNK 256          // k per stage: 32 lanes x 8
__device__ __forceinline__ void gs_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void gs_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void gs_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void gs_unpack8(const uint4& raw, float* out) {
  const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}

// Blocks that stay: one block an SM, and every warp on its own walks a list of items (a tile of up to 4 input rows
// x R weight rows), item after item through one ring of S stages, so that the requests for the next item's first
// chunks are out before the current item ends and the ring stays full across items.  A stage holds one chunk
// (256 k) of the R weight rows and of the tile's input rows (each lane asks for, and later reads, its own 16 bytes of
// every row: no barrier anywhere).  The items of a warp are laid out 32 at a time by its lanes (group, rows and source
// rows of the tile) in shared memory.  Sums per lane in the same order as the forms above, the same tree over lanes.
template <bool GATED, int R, int S>
__global__ void __launch_bounds__(256, 1)
grouped_gemv_walk_kernel(GroupedArgs a, int row_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t gs_smem[];
  constexpr int STAGE = (R + GV_ROWS) * 512;
  constexpr int FEATS = GATED ? R / 2 : R;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* ring = gs_smem + (size_t)warp * S * STAGE + lane * 16;
  int* meta = (int*)(gs_smem + (size_t)8 * S * STAGE) + warp * 32 * 8;
  const bool table = a.tile_group != nullptr;
  const int ncg = (a.N + FEATS - 1) / FEATS;
  const long long n_items = (long long)(table ? a.n_tiles[0] : row_tiles * a.groups) * ncg;
  const int nw = gridDim.x * 8, gw = warp * gridDim.x + blockIdx.x;       // neighbouring items on different SMs
  if (gw >= n_items) return;
  const int my_items = (int)((n_items - gw + nw - 1) / nw);
  const int n_chunks = (a.K + GS_CHUNK - 1) / GS_CHUNK;
  const int kl = lane * 8;
  for (int base = 0; base < my_items; base += 32) {
    const int cnt = min(32, my_items - base);
    if (lane < cnt) {
      const long long item = gw + (long long)(base + lane) * nw;
      const int t = (int)(item / ncg);
      int group, row0, rows;
      if (table) { group = a.tile_group[t]; row0 = a.tile_row0[t]; rows = a.tile_rows[t]; }
      else { group = t / row_tiles; row0 = (t % row_tiles) * GV_ROWS; rows = min(GV_ROWS, a.M - row0); }
      int* m = meta + lane * 8;
      m[0] = group; m[1] = row0; m[2] = rows; m[3] = (int)(item % ncg);
#pragma unroll
      for (int r = 0; r < GV_ROWS; ++r)
        m[4 + r] = r < rows ? (a.row_index != nullptr ? a.row_index[row0 + r] / a.index_div : row0 + r) : -1;
    }
    __syncwarp();
    // the requesting side: item and chunk of the next request, and the item's addresses
    int is_it = 0, is_chunk = 0, is_stage = 0, is_n0 = 0;
    const bf16* is_w = nullptr;
    const bf16* is_x[GV_ROWS] = {};
    auto issue = [&]() {
      if (is_it < cnt) {
        if (is_chunk == 0) {
          const int* m = meta + is_it * 8;
          const int group = m[0];
          is_w = (const bf16*)a.W + (size_t)group * a.w_group_stride;
          is_n0 = m[3] * FEATS;
          const bf16* A = (const bf16*)a.A + (table ? 0 : (size_t)group * a.a_group_off);
#pragma unroll
          for (int r = 0; r < GV_ROWS; ++r) is_x[r] = m[4 + r] >= 0 ? A + (size_t)m[4 + r] * a.lda : nullptr;
        }
        const int k = is_chunk * GS_CHUNK + kl;
        if (k < a.K) {
          uint8_t* st = ring + (size_t)is_stage * STAGE;
#pragma unroll
          for (int j = 0; j < R; ++j) {
            const int n = GATED ? is_n0 + (j >> 1) : is_n0 + j;
            if (n < a.N) gs_cp_async16(st + j * 512, is_w + (size_t)((GATED && (j & 1)) ? a.N + n : n) * a.ldw + k);
          }
#pragma unroll
          for (int r = 0; r < GV_ROWS; ++r)
            if (is_x[r] != nullptr) gs_cp_async16(st + (R + r) * 512, is_x[r] + k);
        }
        if (++is_chunk == n_chunks) { is_chunk = 0; ++is_it; }
      }
      if (++is_stage == S) is_stage = 0;
      gs_commit();                     // one group per request, empty or not: the count stays uniform
    };
#pragma unroll
    for (int c = 0; c < S - 1; ++c) issue();
    float acc[R][GV_ROWS];
    int cp_it = 0, cp_chunk = 0, cp_stage = 0, rows = 0, n0 = 0;
    const int total = cnt * n_chunks;
    for (int i = 0; i < total; ++i) {
      issue();
      gs_wait<S - 1>();                // this lane's requests for step i have landed
      if (cp_chunk == 0) {
#pragma unroll
        for (int j = 0; j < R; ++j)
#pragma unroll
          for (int r = 0; r < GV_ROWS; ++r) acc[j][r] = 0.f;
        rows = meta[cp_it * 8 + 2];
        n0 = meta[cp_it * 8 + 3] * FEATS;
      }
      if (cp_chunk * GS_CHUNK + kl < a.K) {
        const uint8_t* st = ring + (size_t)cp_stage * STAGE;
        auto step = [&](auto nr_tag) {
          constexpr int NR = decltype(nr_tag)::value;
          float x[NR][8];
#pragma unroll
          for (int r = 0; r < NR; ++r) gs_unpack8(*(const uint4*)(st + (R + r) * 512), x[r]);
#pragma unroll
          for (int j = 0; j < R; ++j) {
            if ((GATED ? n0 + (j >> 1) : n0 + j) >= a.N) continue;
            float w[8];
            gs_unpack8(*(const uint4*)(st + j * 512), w);
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[j][r] = fmaf(w[e], x[r][e], acc[j][r]);
          }
        };
        if (rows <= 1) step(std::integral_constant<int, 1>{});
        else if (rows == 2) step(std::integral_constant<int, 2>{});
        else if (rows == 3) step(std::integral_constant<int, 3>{});
        else step(std::integral_constant<int, GV_ROWS>{});
      }
      if (++cp_stage == S) cp_stage = 0;
      if (++cp_chunk == n_chunks) {
#pragma unroll
        for (int j = 0; j < R; ++j)
#pragma unroll
          for (int r = 0; r < GV_ROWS; ++r) acc[j][r] = warp_sum(acc[j][r]);
        if (lane == 0) {
          const int group = meta[cp_it * 8], row0 = meta[cp_it * 8 + 1];
#pragma unroll
          for (int r = 0; r < GV_ROWS; ++r) {
            if (r >= rows) continue;
            const size_t crow = (size_t)(row0 + r) * a.ldc + (table ? 0 : (size_t)group * a.c_group_off);
            if (GATED) {
#pragma unroll
              for (int f = 0; f < R / 2; ++f) {
                const int n = n0 + f;
                if (n >= a.N) continue;
                const float g = fminf(acc[2 * f][r], a.limit);
                const float u = fminf(fmaxf(acc[2 * f + 1][r], -a.limit), a.limit);
                ((bf16*)a.C)[crow + n] = from_f<bf16>(g / (1.f + expf(-a.alpha * g)) * (u + 1.f));
              }
            } else {
#pragma unroll
              for (int j = 0; j < R; ++j) {
                const int n = n0 + j;
                if (n >= a.N) continue;
                if (a.epi == 1) ((float*)a.C)[crow + n] = acc[j][r];
                else ((bf16*)a.C)[crow + n] = from_f<bf16>(grouped_act(acc[j][r], a.epi));
              }
            }
          }
        }
        cp_chunk = 0; ++cp_it;
      }
    }
    gs_wait<0>();
    __syncwarp();                      // the next 32 items overwrite the list
  }
}

// max_tiles: with a tile table, the most tiles the table can hold (the grid's width); tm: 16 or 64 (the
// table must have been built for the same tm); tm = 4 asks for the form for few rows, which needs aligned
// operands (odi_grouped_gemm_takes_few_rows says whether it can run).
static bool vector_loads(const GroupedArgs& a) {
  return a.K % 8 == 0 && a.lda % 8 == 0 && a.ldw % 8 == 0 && a.a_group_off % 8 == 0 && a.w_group_stride % 8 == 0 &&
         (uintptr_t)a.A % 16 == 0 && (uintptr_t)a.W % 16 == 0;
}

extern "C" int odi_grouped_gemm_takes_few_rows(const GroupedArgs* args) {
  return vector_loads(*args) && (size_t)GV_ROWS * args->K * sizeof(float) <= 200 * 1024;
}

extern "C" int odi_grouped_gemm(const GroupedArgs* args, int max_tiles, int tm, int dtype, cudaStream_t stream) {
  const GroupedArgs a = *args;
  if (a.N <= 0 || a.groups <= 0) return 0;
  if (a.K <= 0 || (tm != GV_ROWS && tm != 16 && tm != 64) || a.epi < 0 || a.epi > 5) return ODI_ERR_ARGUMENT;
  if (tm == GV_ROWS) {
    if (!odi_grouped_gemm_takes_few_rows(args)) return ODI_ERR_UNSUPPORTED;
    dim3 grid;
    const int per_block = a.epi == 2 ? 32 : 64;
    if (a.tile_group != nullptr) {
      if (max_tiles <= 0) return 0;
      grid = dim3(max_tiles, (a.N + per_block - 1) / per_block, 1);
    } else {
      if (a.M <= 0) return 0;
      grid = dim3((a.M + GV_ROWS - 1) / GV_ROWS, (a.N + per_block - 1) / per_block, a.groups);
      if (grid.z > 65535) return ODI_ERR_UNSUPPORTED;
    }
    if (grid.y > 65535) return ODI_ERR_UNSUPPORTED;
    const char* form = getenv("ODI_GROUPED_GEMV");
    if (dtype == 1 && (form == nullptr || strcmp(form, "registers") != 0)) {
      // bf16: the weights through a cp.async ring (ODI_GROUPED_GEMV=registers keeps the form above)
      static int sms = 0;
      if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
          sms = 0;
          return ODI_ERR_UNSUPPORTED;
        }
      }
      const int per_feat = a.epi == 2 ? 2 : 1;            // weight rows a feature takes
      const int row_tiles = a.tile_group != nullptr ? 0 : (a.M + GV_ROWS - 1) / GV_ROWS;
      const long long tiles = a.tile_group != nullptr ? max_tiles : (long long)row_tiles * a.groups;
      if (tiles * ((a.N + 1) / 2 + 1) > (1ll << 40)) return ODI_ERR_UNSUPPORTED;
      // items of 8 weight rows ask in larger pieces; items of 4 spread a short list more evenly over the warps
      const long long items8 = tiles * ((a.N * per_feat + 7) / 8);
      const bool wide = form != nullptr ? strcmp(form, "walk8") == 0 : items8 >= 10ll * 8 * sms;
      const int feats = (wide ? 8 : 4) / per_feat;
      const long long items = tiles * ((a.N + feats - 1) / feats);
      const int blocks = (int)std::min<long long>(sms, (items + 7) / 8);
      const size_t walk_smem = (size_t)8 * 6 * (4 + GV_ROWS) * 512 + 8 * 32 * 8 * sizeof(int);   // equal for both shapes
#define ODI_GW(G, R, S) \
      do { cudaError_t e = cudaFuncSetAttribute(grouped_gemv_walk_kernel<G, R, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)walk_smem); \
           if (e != cudaSuccess) return (int)e; \
           odi_rc = launch_pdl((grouped_gemv_walk_kernel<G, R, S>), dim3(blocks), dim3(256), walk_smem, stream, a, row_tiles); } while (0)
      if (wide) { if (a.epi == 2) ODI_GW(true, 8, 4); else ODI_GW(false, 8, 4); }
      else { if (a.epi == 2) ODI_GW(true, 4, 6); else ODI_GW(false, 4, 6); }
#undef ODI_GW
      return launch_status();
    }
    const size_t smem = (size_t)GV_ROWS * a.K * sizeof(float);
#define ODI_GV(T, G) \
    do { cudaError_t e = cudaFuncSetAttribute(grouped_gemv_kernel<T, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
         if (e != cudaSuccess) return (int)e; \
         odi_rc = launch_pdl((grouped_gemv_kernel<T, G>), grid, dim3(256), smem, stream, a); } while (0)
    const bool g = a.epi == 2;
    if (dtype == 0) { if (g) ODI_GV(float, true); else ODI_GV(float, false); }
    else { if (g) ODI_GV(bf16, true); else ODI_GV(bf16, false); }
#undef ODI_GV
    return launch_status();
  }
  dim3 grid;
  if (a.tile_group != nullptr) {
    if (max_tiles <= 0) return 0;
    grid = dim3(max_tiles, (a.N + TN - 1) / TN, 1);
  } else {
    if (a.M <= 0) return 0;
    grid = dim3((a.M + tm - 1) / tm, (a.N + TN - 1) / TN, a.groups);
    if (grid.z > 65535) return ODI_ERR_UNSUPPORTED;
  }
  if (grid.y > 65535) return ODI_ERR_UNSUPPORTED;
  const bool vec = vector_loads(a);
#define ODI_GG(T, TM, G) \
  do { if (vec) odi_rc = launch_pdl((grouped_gemm_kernel<T, TM, G, true>), grid, dim3(256), 0, stream, a); \
       else odi_rc = launch_pdl((grouped_gemm_kernel<T, TM, G, false>), grid, dim3(256), 0, stream, a); } while (0)
  const bool gated = a.epi == 2;
  if (dtype == 0) {
    if (tm == 64) { if (gated) ODI_GG(float, 64, true); else ODI_GG(float, 64, false); }
    else { if (gated) ODI_GG(float, 16, true); else ODI_GG(float, 16, false); }
  } else {
    if (tm == 64) { if (gated) ODI_GG(bf16, 64, true); else ODI_GG(bf16, 64, false); }
    else { if (gated) ODI_GG(bf16, 16, true); else ODI_GG(bf16, 16, false); }
  }
#undef ODI_GG
  return launch_status();
}
