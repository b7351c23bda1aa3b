// Routing of a mixture of experts and the bookkeeping around its grouped products.  Everything here is fp32
// and integer work; nothing waits for the host, so a step with routed experts can be captured in a graph.
//
//  route    per token: scores s = softmax(logits) over all router outputs (or, with `sigmoid`, s_e = 1 / (1 + e^-z_e),
//           each output for itself); choice scores c = s + correction;
//           the router outputs form `n_groups` equal groups of neighbours, a group's score is its largest c,
//           only members of the `keep` best groups may be chosen; the `top` largest c among them are chosen
//           (ties: the lower index); the weight of a chosen output is its s (no renormalisation).
//  table    routing without a router: a token's choices are row `token id` of an integer table, each with the
//           same weight (out-of-range entries take no place).
//  count    per (token, choice) pair whose output is a real expert: its rank among the pairs of that expert.
//  plan     one warp: the experts' offsets in the sorted order of pairs and the table of row tiles.
//           (A step of few pairs does count, plan and scatter in one block and one launch.)
//  scatter  per pair: its place in the sorted order (`pos`) and the order itself (`perm`).
//  combine  per token: residual += sum over its choices, in the order of the choices, of weight times the
//           expert's output row -- or times the token's own input for an identity output (index >= n_experts).
//  gather   the routed tokens' input rows in the sorted order (for products that want their rows side by side).
//  gated_clamp  the experts' activation on a [tokens, 2 F] product (gate lanes, then up lanes):
//           g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1).
#include "common.cuh"

struct RouteArgs {
  const float* logits;      // [n_tokens, n_all]
  const float* correction;  // [n_all] or null
  int* ids;                 // [n_tokens, top]
  float* weights;           // [n_tokens, top]
  int n_tokens, n_all, n_groups, keep, top;
  int sigmoid;              // 1: the score of an output is the logistic function of its logit, not the softmax
};

// (value, index) with "larger value, then lower index" as the order
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// One warp per token; shared memory: per warp n_all scores, n_all choice scores, n_groups group scores.
__global__ void __launch_bounds__(128)
moe_route_kernel(RouteArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * 4 + warp;
  if (t >= a.n_tokens) return;
  float* s = sm + (size_t)warp * (2 * a.n_all + a.n_groups);
  float* c = s + a.n_all;
  float* gs = c + a.n_all;
  const float* z = a.logits + (size_t)t * a.n_all;
  float sum = 1.f;
  if (a.sigmoid) {
    for (int e = lane; e < a.n_all; e += 32) s[e] = 1.0f / (1.0f + expf(-z[e]));
  } else {
    float m = -INFINITY;
    for (int e = lane; e < a.n_all; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    sum = 0.f;
    for (int e = lane; e < a.n_all; e += 32) { const float p = expf(z[e] - m); s[e] = p; sum += p; }
    sum = warp_sum(sum);
  }
  for (int e = lane; e < a.n_all; e += 32) {
    if (!a.sigmoid) s[e] = s[e] / sum;
    c[e] = s[e] + (a.correction != nullptr ? a.correction[e] : 0.f);
  }
  __syncwarp();
  const int per = a.n_all / a.n_groups;
  if (a.keep < a.n_groups) {
    for (int g = lane; g < a.n_groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
      gs[g] = best;
    }
    __syncwarp();
    // mark the `keep` best groups by setting their score to +inf, then drop the members of the others
    for (int k = 0; k < a.keep; ++k) {
      float v = -INFINITY; int i = 0x7fffffff;
      for (int g = lane; g < a.n_groups; g += 32)
        if (gs[g] != INFINITY && (gs[g] > v || (gs[g] == v && g < i))) { v = gs[g]; i = g; }
      warp_argmax(v, i);
      if (lane == 0 && i != 0x7fffffff) gs[i] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < a.n_all; e += 32)
      if (gs[e / per] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < a.top; ++k) {
    float v = -INFINITY; int i = 0x7fffffff;
    for (int e = lane; e < a.n_all; e += 32) {
      const float ce = c[e];
      if (ce != -INFINITY && (i == 0x7fffffff || ce > v)) { v = ce; i = e; }   // -inf: not a candidate
    }
    warp_argmax(v, i);
    if (lane == 0) {
      const bool found = i != 0x7fffffff && v != -INFINITY;
      a.ids[(size_t)t * a.top + k] = found ? i : -1;
      a.weights[(size_t)t * a.top + k] = found ? s[i] : 0.f;
      if (found) c[i] = -INFINITY;
    }
    __syncwarp();
  }
}

extern "C" int odi_moe_route(const RouteArgs* args, cudaStream_t stream) {
  const RouteArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (a.n_all <= 0 || a.n_groups <= 0 || a.n_all % a.n_groups != 0 || a.keep <= 0 || a.keep > a.n_groups || a.top <= 0)
    return ODI_ERR_ARGUMENT;
  const size_t smem = sizeof(float) * 4 * (2 * (size_t)a.n_all + a.n_groups);
  if (smem > 48 * 1024) return ODI_ERR_UNSUPPORTED;
  odi_rc = launch_pdl(moe_route_kernel, dim3((a.n_tokens + 3) / 4), dim3(128), smem, stream, a);
  return launch_status();
}

// ids[t, k] = table[token[t], k] (an entry outside [0, n_experts) becomes -1), weights[t, k] = weight.
__global__ void moe_table_route_kernel(const int* __restrict__ table, const int* __restrict__ tokens, int* __restrict__ ids,
                                       float* __restrict__ weights, int n_pairs, int top, int vocab, int n_experts,
                                       float weight) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  const int token = tokens[p / top];
  int e = -1;
  if (token >= 0 && token < vocab) e = table[(size_t)token * top + p % top];
  if (e < 0 || e >= n_experts) e = -1;
  ids[p] = e;
  weights[p] = weight;
}

extern "C" int odi_moe_table_route(const int* table, const int* tokens, int* ids, float* weights, int n_tokens, int top,
                                   int vocab, int n_experts, float weight, cudaStream_t stream) {
  const int n_pairs = n_tokens * top;
  if (n_pairs <= 0) return 0;
  if (top <= 0 || vocab <= 0 || n_experts <= 0) return ODI_ERR_ARGUMENT;
  odi_rc = launch_pdl(moe_table_route_kernel, dim3((n_pairs + 127) / 128), dim3(128), 0, stream, table, tokens, ids, weights,
                      n_pairs, top, vocab, n_experts, weight);
  return launch_status();
}

struct GroupingArgs {
  const int* ids;     // [n_pairs] chosen output per pair (pair = token * top + choice); -1: none
  int* counts;        // [n_experts], zero on entry; zero again when plan has run
  int* rank;          // [n_pairs]
  int* offsets;       // [n_experts + 1]
  int* pos;           // [n_pairs] place of the pair in the sorted order (undefined for identity outputs)
  int* perm;          // [n_pairs] the sorted order: perm[place] = pair
  int* tile_group;    // [max_tiles]
  int* tile_row0;
  int* tile_rows;
  int* n_tiles;       // [1]
  int n_pairs, n_experts, tm, max_tiles;
};

__global__ void moe_count_kernel(GroupingArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= a.n_pairs) return;
  const int e = a.ids[p];
  if (e >= 0 && e < a.n_experts) a.rank[p] = atomicAdd(&a.counts[e], 1);
}

// One warp: experts 32 at a time, their offsets and tile counts by prefix sums over the lanes, every lane then
// writes the tiles of its own expert.
__global__ void moe_plan_kernel(GroupingArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x;
  int off = 0, tiles = 0;                       // running totals, the same in every lane
  for (int e0 = 0; e0 < a.n_experts; e0 += 32) {
    const int e = e0 + lane;
    const int c = e < a.n_experts ? a.counts[e] : 0;
    if (e < a.n_experts) a.counts[e] = 0;
    const int t = (c + a.tm - 1) / a.tm;
    int c_in = c, t_in = t;                     // inclusive prefix sums
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int cu = __shfl_up_sync(0xffffffffu, c_in, o), tu = __shfl_up_sync(0xffffffffu, t_in, o);
      if (lane >= o) { c_in += cu; t_in += tu; }
    }
    const int my_off = off + c_in - c;
    int my_tile = tiles + t_in - t;
    if (e < a.n_experts) {
      a.offsets[e] = my_off;
      for (int r = 0; r < c && my_tile < a.max_tiles; r += a.tm, ++my_tile) {
        a.tile_group[my_tile] = e; a.tile_row0[my_tile] = my_off + r; a.tile_rows[my_tile] = min(a.tm, c - r);
      }
    }
    off += __shfl_sync(0xffffffffu, c_in, 31);
    tiles += __shfl_sync(0xffffffffu, t_in, 31);
  }
  if (lane == 0) {
    a.offsets[a.n_experts] = off;
    a.n_tiles[0] = min(tiles, a.max_tiles);
  }
}

// Few pairs (single-token steps): count, plan and scatter by one block in one launch, the counts in shared memory
// (the global `counts` stay zero).  Up to SMALL_PAIRS pairs; shared memory holds 2 * n_experts + 1 ints.
#define SMALL_PAIRS 2048
__global__ void __launch_bounds__(256)
moe_group_small_kernel(GroupingArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int sh[];
  int* cnt = sh;
  int* offs = sh + a.n_experts;
  const int tid = threadIdx.x;
  for (int e = tid; e < a.n_experts; e += 256) cnt[e] = 0;
  __syncthreads();
  int my_e[SMALL_PAIRS / 256], my_rank[SMALL_PAIRS / 256];
#pragma unroll
  for (int j = 0; j < SMALL_PAIRS / 256; ++j) {
    const int p = tid + j * 256;
    my_e[j] = -1;
    if (p < a.n_pairs) {
      const int e = a.ids[p];
      if (e >= 0 && e < a.n_experts) { my_e[j] = e; my_rank[j] = atomicAdd(&cnt[e], 1); }
    }
  }
  __syncthreads();
  if (tid < 32) {
    // the same walk as moe_plan_kernel, over the counts in shared memory
    int off = 0, tiles = 0;
    for (int e0 = 0; e0 < a.n_experts; e0 += 32) {
      const int e = e0 + tid;
      const int c = e < a.n_experts ? cnt[e] : 0;
      const int t = (c + a.tm - 1) / a.tm;
      int c_in = c, t_in = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int cu = __shfl_up_sync(0xffffffffu, c_in, o), tu = __shfl_up_sync(0xffffffffu, t_in, o);
        if (tid >= o) { c_in += cu; t_in += tu; }
      }
      const int my_off = off + c_in - c;
      int my_tile = tiles + t_in - t;
      if (e < a.n_experts) {
        offs[e] = my_off;
        a.offsets[e] = my_off;
        for (int r = 0; r < c && my_tile < a.max_tiles; r += a.tm, ++my_tile) {
          a.tile_group[my_tile] = e; a.tile_row0[my_tile] = my_off + r; a.tile_rows[my_tile] = min(a.tm, c - r);
        }
      }
      off += __shfl_sync(0xffffffffu, c_in, 31);
      tiles += __shfl_sync(0xffffffffu, t_in, 31);
    }
    if (tid == 0) {
      a.offsets[a.n_experts] = off;
      a.n_tiles[0] = min(tiles, a.max_tiles);
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < SMALL_PAIRS / 256; ++j) {
    const int p = tid + j * 256;
    if (my_e[j] >= 0) {
      const int place = offs[my_e[j]] + my_rank[j];
      a.rank[p] = my_rank[j];
      a.pos[p] = place;
      a.perm[place] = p;
    }
  }
}

__global__ void moe_scatter_kernel(GroupingArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= a.n_pairs) return;
  const int e = a.ids[p];
  if (e >= 0 && e < a.n_experts) {
    const int place = a.offsets[e] + a.rank[p];
    a.pos[p] = place;
    a.perm[place] = p;
  }
}

extern "C" int odi_moe_group(const GroupingArgs* args, cudaStream_t stream) {
  const GroupingArgs a = *args;
  if (a.n_pairs <= 0) return 0;
  if (a.n_experts <= 0 || a.tm <= 0 || a.max_tiles < (a.n_pairs + a.tm - 1) / a.tm + a.n_experts) return ODI_ERR_ARGUMENT;
  if (a.n_pairs <= SMALL_PAIRS && a.n_experts <= 4096) {
    odi_rc = launch_pdl(moe_group_small_kernel, dim3(1), dim3(256), sizeof(int) * (2 * (size_t)a.n_experts + 1), stream, a);
    return launch_status();
  }
  const int blocks = (a.n_pairs + 255) / 256;
  odi_rc = launch_pdl(moe_count_kernel, dim3(blocks), dim3(256), 0, stream, a);
  if (odi_rc == 0) odi_rc = launch_pdl(moe_plan_kernel, dim3(1), dim3(32), 0, stream, a);
  if (odi_rc == 0) odi_rc = launch_pdl(moe_scatter_kernel, dim3(blocks), dim3(256), 0, stream, a);
  return launch_status();
}

struct CombineArgs {
  float* residual;        // [n_tokens, H], added to in place
  const void* expert_out;   // [n_pairs, H] rows in the sorted order: fp32, or T if out_is_t
  const void* input;      // [n_tokens, H] in T: what identity outputs pass on
  const int* ids;
  const float* weights;   // null: every chosen row counts once (the weights were applied elsewhere)
  const int* pos;
  int n_tokens, H, top, n_experts, out_is_t;
  int assign;             // the sums replace the rows of `residual` instead of being added to them
};

template <typename T>
__global__ void moe_combine_kernel(CombineArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < a.H; i += gridDim.y * blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < a.top; ++k) {
      const int p = t * a.top + k;
      const int e = a.ids[p];
      if (e < 0) continue;
      float v;
      if (e >= a.n_experts) v = to_f<T>(((const T*)a.input)[(size_t)t * a.H + i]);
      else if (a.out_is_t) v = to_f<T>(((const T*)a.expert_out)[(size_t)a.pos[p] * a.H + i]);
      else v = ((const float*)a.expert_out)[(size_t)a.pos[p] * a.H + i];
      sum = fmaf(a.weights != nullptr ? a.weights[p] : 1.f, v, sum);
    }
    if (a.assign) a.residual[(size_t)t * a.H + i] = sum;
    else a.residual[(size_t)t * a.H + i] += sum;
  }
}

// bf16 inputs, eight lanes per thread (H a multiple of 8, aligned rows): the same sums in the same order.
__global__ void moe_combine_vec_kernel(CombineArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < a.H; i += gridDim.y * blockDim.x * 8) {
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < a.top; ++k) {
      const int p = t * a.top + k;
      const int e = a.ids[p];
      if (e < 0) continue;
      float v[8];
      if (e < a.n_experts && !a.out_is_t) {
        const float* src = (const float*)a.expert_out + (size_t)a.pos[p] * a.H + i;
        const float4 lo = *(const float4*)src, hi = *(const float4*)(src + 4);
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      } else {
        const bf16* src = e >= a.n_experts ? (const bf16*)a.input + (size_t)t * a.H + i
                                           : (const bf16*)a.expert_out + (size_t)a.pos[p] * a.H + i;
        const uint4 raw = *(const uint4*)src;
        const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw;
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
      }
      const float w = a.weights != nullptr ? a.weights[p] : 1.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) sum[j] = fmaf(w, v[j], sum[j]);
    }
    float4* dst = (float4*)(a.residual + (size_t)t * a.H + i);
    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
    if (!a.assign) { lo = dst[0]; hi = dst[1]; }
    lo.x += sum[0]; lo.y += sum[1]; lo.z += sum[2]; lo.w += sum[3]; hi.x += sum[4]; hi.y += sum[5]; hi.z += sum[6]; hi.w += sum[7];
    dst[0] = lo; dst[1] = hi;
  }
}

extern "C" int odi_moe_combine(const CombineArgs* args, int dtype, cudaStream_t stream) {
  const CombineArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (dtype == 1 && a.H % 8 == 0 && ((uintptr_t)a.residual | (uintptr_t)a.expert_out | (uintptr_t)a.input) % 16 == 0) {
    const int vthreads = a.H >= 2048 ? 256 : (a.H >= 1024 ? 128 : 64);
    const int vpieces = a.n_tokens >= 512 ? 1 : min(8, (a.H / 8 + vthreads - 1) / vthreads);
    odi_rc = launch_pdl(moe_combine_vec_kernel, dim3(a.n_tokens, vpieces), dim3(vthreads), 0, stream, a);
    return launch_status();
  }
  const int threads = a.H >= 1024 ? 256 : 128;
  // few tokens: a row's lanes over several blocks, so that each thread has one short chain of loads
  const int pieces = a.n_tokens >= 512 ? 1 : min(16, (a.H + threads - 1) / threads);
  const dim3 grid(a.n_tokens, pieces);
  if (dtype == 0) odi_rc = launch_pdl((moe_combine_kernel<float>), grid, dim3(threads), 0, stream, a);
  else odi_rc = launch_pdl((moe_combine_kernel<bf16>), grid, dim3(threads), 0, stream, a);
  return launch_status();
}

// Rows of the routed tokens' inputs in the sorted order: out[i] = x[perm[i] / top] for the places that are taken;
// with `weights` ([tokens, top], fp32) the row is multiplied by the weight of its (token, choice) pair, in fp32,
// and rounded once (experts whose weight multiplies their input).
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ perm, const int* __restrict__ offsets,
                                  T* __restrict__ out, int H, int top, int n_experts, const float* __restrict__ weights) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= offsets[n_experts]) return;
  const T* src = x + (size_t)(perm[i] / top) * H;
  T* dst = out + (size_t)i * H;
  if (weights != nullptr) {
    const float w = weights[perm[i]];
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = from_f<T>(w * to_f<T>(src[c]));
    return;
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = src[c];
}

// The same in pieces of 16 bytes (row_bytes a multiple of 16, aligned rows).
__global__ void moe_gather_vec_kernel(const uint4* __restrict__ x, const int* __restrict__ perm, const int* __restrict__ offsets,
                                      uint4* __restrict__ out, int row16, int top, int n_experts) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= offsets[n_experts]) return;
  const uint4* src = x + (size_t)(perm[i] / top) * row16;
  uint4* dst = out + (size_t)i * row16;
  for (int c = threadIdx.x; c < row16; c += blockDim.x) dst[c] = src[c];
}

extern "C" int odi_moe_gather(const void* x, const int* perm, const int* offsets, void* out, int n_pairs, int H, int top,
                              int n_experts, const float* weights, int dtype, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  const size_t row_bytes = (size_t)H * (dtype == 0 ? 4 : 2);
  if (weights == nullptr && row_bytes % 16 == 0 && ((uintptr_t)x | (uintptr_t)out) % 16 == 0) {
    const int row16 = (int)(row_bytes / 16);
    odi_rc = launch_pdl(moe_gather_vec_kernel, dim3(n_pairs), dim3(row16 >= 256 ? 256 : 128), 0, stream, (const uint4*)x, perm, offsets, (uint4*)out, row16, top, n_experts);
    return launch_status();
  }
  if (dtype == 0) odi_rc = launch_pdl((moe_gather_kernel<float>), dim3(n_pairs), dim3(128), 0, stream, (const float*)x, perm, offsets, (float*)out, H, top, n_experts, weights);
  else odi_rc = launch_pdl((moe_gather_kernel<bf16>), dim3(n_pairs), dim3(128), 0, stream, (const bf16*)x, perm, offsets, (bf16*)out, H, top, n_experts, weights);
  return launch_status();
}

template <typename T>
__global__ void gated_clamp_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long n, int F, float limit,
                                   float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long row = i / F;
  const int f = (int)(i % F);
  const float g = fminf(to_f<T>(gate_up[row * 2 * F + f]), limit);
  const float u = fminf(fmaxf(to_f<T>(gate_up[row * 2 * F + F + f]), -limit), limit);
  out[i] = from_f<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

// bf16, eight lanes a thread (F a multiple of 8, aligned rows): the same arithmetic.
__global__ void gated_clamp_vec_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, long long n8, int F, float limit,
                                       float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i8 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i8 >= n8) return;
  const long long i = i8 * 8, row = i / F;
  const int f = (int)(i % F);
  const uint4 graw = *(const uint4*)(gate_up + row * 2 * F + f), uraw = *(const uint4*)(gate_up + row * 2 * F + F + f);
  const __nv_bfloat162* g2 = (const __nv_bfloat162*)&graw;
  const __nv_bfloat162* u2 = (const __nv_bfloat162*)&uraw;
  uint4 oraw;
  __nv_bfloat162* o2 = (__nv_bfloat162*)&oraw;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 gv = __bfloat1622float2(g2[e]), uv = __bfloat1622float2(u2[e]);
    const float g0 = fminf(gv.x, limit), g1 = fminf(gv.y, limit);
    const float u0 = fminf(fmaxf(uv.x, -limit), limit), u1 = fminf(fmaxf(uv.y, -limit), limit);
    o2[e] = __floats2bfloat162_rn(g0 / (1.f + expf(-alpha * g0)) * (u0 + 1.f), g1 / (1.f + expf(-alpha * g1)) * (u1 + 1.f));
  }
  *(uint4*)(out + i) = oraw;
}

extern "C" int odi_gated_clamp(const void* gate_up, void* out, int rows, int F, float limit, float alpha, int dtype,
                               cudaStream_t stream) {
  const long long n = (long long)rows * F;
  if (n <= 0) return 0;
  if (dtype == 1 && F % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
    const long long n8 = n / 8;
    odi_rc = launch_pdl(gated_clamp_vec_kernel, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, stream, (const bf16*)gate_up,
                        (bf16*)out, n8, F, limit, alpha);
    return launch_status();
  }
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == 0) odi_rc = launch_pdl((gated_clamp_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)out, n, F, limit, alpha);
  else odi_rc = launch_pdl((gated_clamp_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, n, F, limit, alpha);
  return launch_status();
}
