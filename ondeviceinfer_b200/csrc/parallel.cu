// Kernels of a block whose mixer and feed-forward read ONE norm of the stream side by side,
//   h = norm(x);  x <- x + m (mixer(h + conv(h)) + ff(h)),
// with a short causal convolution over time in front of the mixer, and of a feed-forward whose activation is a
// polynomial of row-normed powers:
//
//  * canon_norm: per token the norm of its row (one number g as the weight), h in T for the feed-forward, and
//    h + conv(h) in T for the mixer, conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j).  The rows before t come from
//    the step's own tokens (their norm is taken again: the rows are in L2) or, before the first token that a
//    sequence brings, from the sequence's state: h of its last taps - 1 positions, fp32, zero before its start.
//    A sequence that brings one token has its state moved on in the same launch (the thread that reads a channel's
//    state rows writes them back shifted).  For many tokens a block takes a run of them, so that a row's norm is
//    taken once per run instead of once per tap.
//  * canon_state: afterwards, the state of every sequence that brought more than one token moved on by them.
//  * poly_norm: out = a N(z) + b N(z^2) + c N(z^3) + e, N(v) = v / sqrt(mean(v^2) + eps) over a token's row.
//  * scaled_add: x += m y on fp32 rows.
// Norms, the convolution's sum and the powers are fp32 in both compute dtypes; each output is rounded once.
#include "common.cuh"

#define CANON_MAX_TAPS 8          // the forms with 16-byte accesses keep the taps' factors in registers
#define CANON_MOST_TAPS 64        // the plain form keeps them in shared memory

struct CanonArgs {
  const float* x;        // [n_tokens, W] the stream
  const float* g;        // one number
  const float* taps_w;   // [W, taps]
  float* state;          // [slots, taps - 1, W]; null when taps == 1
  const int* tok_seq;    // [n_tokens]
  const int* cu_q;       // [n_seqs + 1]
  const int* slots;      // [n_seqs]
  void* h_out;           // [n_tokens, W] in T
  void* hc_out;          // [n_tokens, W] in T
  int n_tokens, n_seqs, W, taps;
  float eps;
};

template <typename T>
__global__ void __launch_bounds__(256)
canon_norm_kernel(CanonArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  __shared__ float inv[CANON_MOST_TAPS];
  const int t = blockIdx.x;
  const int seq = a.tok_seq[t];
  const int i = t - a.cu_q[seq];            // index among the tokens that the sequence brings in this step
  const int W = a.W, taps = a.taps;
  const float g = a.g[0];
  for (int k = 0; k < taps && i - k >= 0; ++k) {
    const float* xr = a.x + (size_t)(t - k) * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float v = xr[c]; ss += v * v; }
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) inv[k] = g / sqrtf(ss / (float)W + a.eps);
  }
  __syncthreads();
  const float* st = a.state != nullptr ? a.state + (size_t)a.slots[seq] * (taps - 1) * W : nullptr;
  const bool single = st != nullptr && a.cu_q[seq + 1] - a.cu_q[seq] == 1;
  T* h = (T*)a.h_out + (size_t)t * W;
  T* hc = (T*)a.hc_out + (size_t)t * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float h0 = a.x[(size_t)t * W + c] * inv[0];
    const float* w = a.taps_w + (size_t)c * taps;
    float acc = h0 * w[taps - 1];
    for (int k = 1; k < taps; ++k) {
      // position t - k: a token of this step, or row (taps - 1) + (i - k) of the state
      const float hk = i - k >= 0 ? a.x[(size_t)(t - k) * W + c] * inv[k] : st[(size_t)(taps - 1 + i - k) * W + c];
      acc = fmaf(hk, w[taps - 1 - k], acc);
    }
    h[c] = from_f<T>(h0);
    hc[c] = from_f<T>(h0 + acc);
    if (single) {      // a sequence of one token: its state moves on here (this thread alone touches the channel)
      float* sw = a.state + (size_t)a.slots[seq] * (taps - 1) * W;
      for (int j = 0; j + 2 < taps; ++j) sw[(size_t)j * W + c] = sw[(size_t)(j + 1) * W + c];
      sw[(size_t)(taps - 2) * W + c] = h0;
    }
  }
}

// Sums of up to CANON_MAX_TAPS values over the block at once (one pair of barriers); every thread gets them.
__device__ __forceinline__ void block_sum_taps(float* v, int count, float (*scratch)[33]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int k = 0; k < CANON_MAX_TAPS; ++k) if (k < count) v[k] = warp_sum(v[k]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < CANON_MAX_TAPS; ++k) if (k < count) scratch[k][warp] = v[k];
  }
  __syncthreads();
  if (warp < count) {
    float t = lane < nwarps ? scratch[warp][lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[warp][32] = t;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < CANON_MAX_TAPS; ++k) if (k < count) v[k] = scratch[k][32];
}

template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *(float4*)p = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
  uint2 packed;
  *(__nv_bfloat162*)&packed.x = __floats2bfloat162_rn(a, b);
  *(__nv_bfloat162*)&packed.y = __floats2bfloat162_rn(c, d);
  *(uint2*)p = packed;
}

// The same for widths that are multiples of 4 (and blocks of at least as many warps as taps): 16-byte loads of the stream,
// all rows' sums of squares in one reduction, 8- or 16-byte stores.  TAPS is the number of taps (a template argument
// so that the rows' factors stay in registers).
template <typename T, int TAPS>
__global__ void __launch_bounds__(256)
canon_norm_vec_kernel(CanonArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[CANON_MAX_TAPS][33];
  const int t = blockIdx.x;
  const int seq = a.tok_seq[t];
  const int i = t - a.cu_q[seq];
  const int W = a.W, W4 = W >> 2;
  const float g = a.g[0];
  const float4* x4 = (const float4*)a.x;
  float ss[CANON_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < CANON_MAX_TAPS; ++k) ss[k] = 0.f;
  for (int c = threadIdx.x; c < W4; c += blockDim.x) {
#pragma unroll
    for (int k = 0; k < TAPS; ++k) {
      if (i - k >= 0) {
        const float4 v = x4[(size_t)(t - k) * W4 + c];
        ss[k] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    }
  }
  block_sum_taps(ss, TAPS, scratch);
  float inv[TAPS];
#pragma unroll
  for (int k = 0; k < TAPS; ++k) inv[k] = g / sqrtf(ss[k] / (float)W + a.eps);
  const float4* st4 = a.state != nullptr ? (const float4*)(a.state + (size_t)a.slots[seq] * (TAPS - 1) * W) : nullptr;
  const bool single = TAPS > 1 && st4 != nullptr && a.cu_q[seq + 1] - a.cu_q[seq] == 1;
  T* h = (T*)a.h_out + (size_t)t * W;
  T* hc = (T*)a.hc_out + (size_t)t * W;
  for (int c = threadIdx.x; c < W4; c += blockDim.x) {
    float4 v = x4[(size_t)t * W4 + c];
    const float h0[4] = {v.x * inv[0], v.y * inv[0], v.z * inv[0], v.w * inv[0]};
    float w[4][TAPS];
    if (TAPS % 4 == 0) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int j = 0; j < TAPS; j += 4) {
          const float4 q = *(const float4*)(a.taps_w + (size_t)(4 * c + e) * TAPS + j);
          w[e][j] = q.x; w[e][j + 1] = q.y; w[e][j + 2] = q.z; w[e][j + 3] = q.w;
        }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) w[e][j] = a.taps_w[(size_t)(4 * c + e) * TAPS + j];
    }
    float acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] = h0[e] * w[e][TAPS - 1];
    float4 before[TAPS];       // h of position t - k
#pragma unroll
    for (int k = 1; k < TAPS; ++k) {
      float4 r;
      if (i - k >= 0) {
        r = x4[(size_t)(t - k) * W4 + c];
        r.x *= inv[k]; r.y *= inv[k]; r.z *= inv[k]; r.w *= inv[k];
      } else {
        r = st4[(size_t)(TAPS - 1 + i - k) * W4 + c];
      }
      before[k] = r;
      acc[0] = fmaf(r.x, w[0][TAPS - 1 - k], acc[0]); acc[1] = fmaf(r.y, w[1][TAPS - 1 - k], acc[1]);
      acc[2] = fmaf(r.z, w[2][TAPS - 1 - k], acc[2]); acc[3] = fmaf(r.w, w[3][TAPS - 1 - k], acc[3]);
    }
    store4<T>(h + 4 * c, h0[0], h0[1], h0[2], h0[3]);
    store4<T>(hc + 4 * c, h0[0] + acc[0], h0[1] + acc[1], h0[2] + acc[2], h0[3] + acc[3]);
    if (single) {      // a sequence of one token: its state moves on here (this thread alone touches the channel)
      float4* sw4 = (float4*)(a.state + (size_t)a.slots[seq] * (TAPS - 1) * W);
#pragma unroll
      for (int j = 0; j + 2 < TAPS; ++j) sw4[(size_t)j * W4 + c] = before[TAPS - 2 - j];
      sw4[(size_t)(TAPS - 2) * W4 + c] = make_float4(h0[0], h0[1], h0[2], h0[3]);
    }
  }
}

// Many tokens: a block takes RUN consecutive tokens of the packed step.  First the factors of the run's rows and of
// the TAPS - 1 rows before it (each row's sum of squares once per block), then every thread walks its channels down
// the run with the last TAPS - 1 rows of h in registers.  A token whose sequence starts inside the run (or whose
// earlier positions are not of this step) takes those rows from the state instead.
template <typename T, int TAPS, int RUN>
__global__ void __launch_bounds__(256)
canon_norm_run_kernel(CanonArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ROWS = RUN + TAPS - 1;
  __shared__ float part[ROWS][8];
  __shared__ float inv_s[ROWS];
  __shared__ int first_s[RUN], slot_s[RUN], single_s[RUN];   // per token: its index among its sequence's tokens of
                                                             // the step, its slot, whether it is the only one
  const int t0 = blockIdx.x * RUN;
  const int W = a.W, W4 = W >> 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float4* x4 = (const float4*)a.x;
  if (threadIdx.x < RUN && t0 + threadIdx.x < a.n_tokens) {
    const int seq = a.tok_seq[t0 + threadIdx.x];
    first_s[threadIdx.x] = t0 + threadIdx.x - a.cu_q[seq];
    slot_s[threadIdx.x] = a.slots[seq];
    single_s[threadIdx.x] = TAPS > 1 && a.cu_q[seq + 1] - a.cu_q[seq] == 1;
  }
  float ss[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) ss[r] = 0.f;
  for (int c = threadIdx.x; c < W4; c += blockDim.x) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int t = t0 - (TAPS - 1) + r;
      if (t >= 0 && t < a.n_tokens) {
        const float4 v = x4[(size_t)t * W4 + c];
        ss[r] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    ss[r] = warp_sum(ss[r]);
    if (lane == 0) part[r][warp] = ss[r];
  }
  __syncthreads();
  if (threadIdx.x < ROWS) {
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += part[threadIdx.x][w];
    inv_s[threadIdx.x] = a.g[0] / sqrtf(s / (float)W + a.eps);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < W4; c += blockDim.x) {
    float w[4][TAPS];          // the taps of channels 4 c to 4 c + 3: 4 TAPS numbers in a row
    {
      float flat[4 * TAPS];
#pragma unroll
      for (int j = 0; j < TAPS; ++j) *(float4*)(flat + 4 * j) = *(const float4*)(a.taps_w + (size_t)4 * c * TAPS + 4 * j);
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) w[e][j] = flat[e * TAPS + j];
    }
    float4 before[TAPS];       // before[k]: h of the packed token k places back
#pragma unroll
    for (int k = 1; k < TAPS; ++k) {
      const int t = t0 - k;
      float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t >= 0) {
        const float f = inv_s[TAPS - 1 - k];
        r = x4[(size_t)t * W4 + c];
        r.x *= f; r.y *= f; r.z *= f; r.w *= f;
      }
      before[k] = r;
    }
#pragma unroll
    for (int j = 0; j < RUN; ++j) {
      const int t = t0 + j;
      if (t < a.n_tokens) {
        const int i = first_s[j];
        const float f = inv_s[TAPS - 1 + j];
        float4 v = x4[(size_t)t * W4 + c];
        v.x *= f; v.y *= f; v.z *= f; v.w *= f;
        float acc[4] = {v.x * w[0][TAPS - 1], v.y * w[1][TAPS - 1], v.z * w[2][TAPS - 1], v.w * w[3][TAPS - 1]};
        float4 used[TAPS];
#pragma unroll
        for (int k = 1; k < TAPS; ++k) {
          float4 r = before[k];
          if (i - k < 0) r = ((const float4*)(a.state + (size_t)slot_s[j] * (TAPS - 1) * W))[(size_t)(TAPS - 1 + i - k) * W4 + c];
          used[k] = r;
          acc[0] = fmaf(r.x, w[0][TAPS - 1 - k], acc[0]); acc[1] = fmaf(r.y, w[1][TAPS - 1 - k], acc[1]);
          acc[2] = fmaf(r.z, w[2][TAPS - 1 - k], acc[2]); acc[3] = fmaf(r.w, w[3][TAPS - 1 - k], acc[3]);
        }
        store4<T>((T*)a.h_out + (size_t)t * W + 4 * c, v.x, v.y, v.z, v.w);
        store4<T>((T*)a.hc_out + (size_t)t * W + 4 * c, v.x + acc[0], v.y + acc[1], v.z + acc[2], v.w + acc[3]);
        if (single_s[j]) {     // a sequence of one token: its state moves on here
          float4* sw4 = (float4*)(a.state + (size_t)slot_s[j] * (TAPS - 1) * W);
#pragma unroll
          for (int r = 0; r + 2 < TAPS; ++r) sw4[(size_t)r * W4 + c] = used[TAPS - 2 - r];
          sw4[(size_t)(TAPS > 1 ? TAPS - 2 : 0) * W4 + c] = v;
        }
#pragma unroll
        for (int k = TAPS - 1; k >= 2; --k) before[k] = before[k - 1];
        before[TAPS > 1 ? 1 : 0] = v;
      }
    }
  }
}

// One block per sequence: row j of the new state is h at index T - (taps - 1) + j of the step's tokens, or, for
// a sequence that brought fewer than taps - 1 tokens, row T + j of the old state (ascending j, each channel by
// one thread, so the move in place is safe).
__global__ void __launch_bounds__(256)
canon_state_kernel(CanonArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int seq = blockIdx.x;
  const int W = a.W, keep = a.taps - 1;
  const int begin = a.cu_q[seq], T = a.cu_q[seq + 1] - begin;
  if (T == 1) return;          // canon_norm moved it on
  const float g = a.g[0];
  float* st = a.state + (size_t)a.slots[seq] * keep * W;
  for (int j = 0; j < keep; ++j) {
    const int i = T - keep + j;
    if (i >= 0) {
      const float* xr = a.x + (size_t)(begin + i) * W;
      float ss = 0.f;
      for (int c = threadIdx.x; c < W; c += blockDim.x) { const float v = xr[c]; ss += v * v; }
      ss = block_sum(ss, scratch);
      const float inv = g / sqrtf(ss / (float)W + a.eps);
      for (int c = threadIdx.x; c < W; c += blockDim.x) st[(size_t)j * W + c] = xr[c] * inv;
    } else {
      for (int c = threadIdx.x; c < W; c += blockDim.x) st[(size_t)j * W + c] = st[(size_t)(T + j) * W + c];
    }
  }
}

// The same with 16-byte accesses and one reduction for all rows (widths that are multiples of 4).
template <int TAPS>
__global__ void __launch_bounds__(256)
canon_state_vec_kernel(CanonArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[CANON_MAX_TAPS][33];
  constexpr int keep = TAPS - 1;
  const int seq = blockIdx.x;
  const int W = a.W, W4 = W >> 2;
  const int begin = a.cu_q[seq], T = a.cu_q[seq + 1] - begin;
  if (T == 1) return;          // canon_norm moved it on
  const float g = a.g[0];
  const float4* x4 = (const float4*)a.x;
  float4* st4 = (float4*)(a.state + (size_t)a.slots[seq] * keep * W);
  float ss[CANON_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < CANON_MAX_TAPS; ++k) ss[k] = 0.f;
  for (int c = threadIdx.x; c < W4; c += blockDim.x) {
#pragma unroll
    for (int j = 0; j < keep; ++j) {
      const int i = T - keep + j;
      if (i >= 0) {
        const float4 v = x4[(size_t)(begin + i) * W4 + c];
        ss[j] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    }
  }
  block_sum_taps(ss, keep, scratch);
  for (int c = threadIdx.x; c < W4; c += blockDim.x) {
#pragma unroll
    for (int j = 0; j < keep; ++j) {
      const int i = T - keep + j;
      float4 v;
      if (i >= 0) {
        const float inv = g / sqrtf(ss[j] / (float)W + a.eps);
        v = x4[(size_t)(begin + i) * W4 + c];
        v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
      } else {
        v = st4[(size_t)(T + j) * W4 + c];
      }
      st4[(size_t)j * W4 + c] = v;
    }
  }
}

extern "C" int odi_canon_norm(const CanonArgs* args, int dtype, cudaStream_t stream) {
  const CanonArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (a.taps < 1 || a.taps > CANON_MOST_TAPS || a.W <= 0 || (a.taps > 1 && a.state == nullptr)) return ODI_ERR_UNSUPPORTED;
  const int threads = a.W >= 1024 ? 256 : 128;
  const bool aligned = a.taps <= CANON_MAX_TAPS && a.W % 4 == 0 &&
                       (((uintptr_t)a.x | (uintptr_t)a.state | (uintptr_t)a.h_out | (uintptr_t)a.hc_out | (uintptr_t)a.taps_w) & 15) == 0;
#define ODI_CANON(T, K) odi_rc = launch_pdl((canon_norm_vec_kernel<T, K>), dim3(a.n_tokens), dim3(threads), 0, stream, a)
#define ODI_CANON_TAPS(T) switch (a.taps) { case 1: ODI_CANON(T, 1); break; case 2: ODI_CANON(T, 2); break; \
    case 3: ODI_CANON(T, 3); break; case 4: ODI_CANON(T, 4); break; case 5: ODI_CANON(T, 5); break; \
    case 6: ODI_CANON(T, 6); break; case 7: ODI_CANON(T, 7); break; default: ODI_CANON(T, 8); break; }
  if (aligned && threads / 32 >= a.taps && a.n_tokens < 512) {
    if (dtype == 0) { ODI_CANON_TAPS(float) } else { ODI_CANON_TAPS(bf16) }
    return launch_status();
  }
#undef ODI_CANON
  if (aligned) {       // many tokens: runs of four, or of eight once those fill the device several times over
    const int run = a.n_tokens < 4096 ? 4 : 8;
#define ODI_CANON(T, K) if (run == 4) odi_rc = launch_pdl((canon_norm_run_kernel<T, K, 4>), dim3((a.n_tokens + 3) / 4), \
        dim3(threads), 0, stream, a); \
    else odi_rc = launch_pdl((canon_norm_run_kernel<T, K, 8>), dim3((a.n_tokens + 7) / 8), dim3(threads), 0, stream, a)
    if (dtype == 0) { ODI_CANON_TAPS(float) } else { ODI_CANON_TAPS(bf16) }
    return launch_status();
  }
#undef ODI_CANON_TAPS
#undef ODI_CANON
  if (dtype == 0) odi_rc = launch_pdl((canon_norm_kernel<float>), dim3(a.n_tokens), dim3(threads), 0, stream, a);
  else odi_rc = launch_pdl((canon_norm_kernel<bf16>), dim3(a.n_tokens), dim3(threads), 0, stream, a);
  return launch_status();
}

extern "C" int odi_canon_state(const CanonArgs* args, cudaStream_t stream) {
  const CanonArgs a = *args;
  if (a.n_seqs <= 0 || a.taps <= 1) return 0;
  if (a.taps > CANON_MOST_TAPS || a.state == nullptr) return ODI_ERR_UNSUPPORTED;
  const int threads = a.W >= 1024 ? 256 : 128;
  if (a.taps <= CANON_MAX_TAPS && a.W % 4 == 0 && (((uintptr_t)a.x | (uintptr_t)a.state) & 15) == 0 && threads / 32 >= a.taps) {
#define ODI_STATE(K) odi_rc = launch_pdl((canon_state_vec_kernel<K>), dim3(a.n_seqs), dim3(threads), 0, stream, a)
    switch (a.taps) {
      case 2: ODI_STATE(2); break; case 3: ODI_STATE(3); break; case 4: ODI_STATE(4); break; case 5: ODI_STATE(5); break;
      case 6: ODI_STATE(6); break; case 7: ODI_STATE(7); break; default: ODI_STATE(8); break;
    }
#undef ODI_STATE
    return launch_status();
  }
  odi_rc = launch_pdl((canon_state_kernel), dim3(a.n_seqs), dim3(threads), 0, stream, a);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// out = a N(z) + b N(z^2) + c N(z^3) + e per row of F lanes; coef = (a, b, c, e) in fp32.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_kernel(const T* __restrict__ z, const float* __restrict__ coef, T* __restrict__ out, int F, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const T* zr = z + (size_t)blockIdx.x * F;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = to_f<T>(zr[i]);
    const float v2 = v * v, v3 = v2 * v;
    s2 += v2; s4 += v2 * v2; s6 += v3 * v3;
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float k1 = coef[0] / sqrtf(s2 / (float)F + eps);
  const float k2 = coef[1] / sqrtf(s4 / (float)F + eps);
  const float k3 = coef[2] / sqrtf(s6 / (float)F + eps);
  const float e = coef[3];
  T* o = out + (size_t)blockIdx.x * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = to_f<T>(zr[i]);
    o[i] = from_f<T>(fmaf(v, fmaf(v, fmaf(v, k3, k2), k1), e));
  }
}

// Eight lanes a step (F a multiple of 8, aligned rows): 16-byte loads of bf16, two of floats.
template <typename T> __device__ __forceinline__ void load8(const T* p, float* v);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* v) {
  const float4 lo = *(const float4*)p, hi = *(const float4*)(p + 4);
  v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* v) {
  const uint4 raw = *(const uint4*)p;
  const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw;
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h2[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* v);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* v) {
  *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
  *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* p, const float* v) {
  uint4 packed;
  __nv_bfloat162* h2 = (__nv_bfloat162*)&packed;
#pragma unroll
  for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *(uint4*)p = packed;
}

template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_vec_kernel(const T* __restrict__ z, const float* __restrict__ coef, T* __restrict__ out, int F, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[CANON_MAX_TAPS][33];
  const T* zr = z + (size_t)blockIdx.x * F;
  float s[CANON_MAX_TAPS] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = threadIdx.x * 8; i < F; i += blockDim.x * 8) {
    float v[8];
    load8<T>(zr + i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float v2 = v[e] * v[e], v3 = v2 * v[e];
      s[0] += v2; s[1] += v2 * v2; s[2] += v3 * v3;
    }
  }
  block_sum_taps(s, 3, scratch);
  const float k1 = coef[0] / sqrtf(s[0] / (float)F + eps);
  const float k2 = coef[1] / sqrtf(s[1] / (float)F + eps);
  const float k3 = coef[2] / sqrtf(s[2] / (float)F + eps);
  const float e0 = coef[3];
  T* o = out + (size_t)blockIdx.x * F;
  for (int i = threadIdx.x * 8; i < F; i += blockDim.x * 8) {
    float v[8];
    load8<T>(zr + i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = fmaf(v[e], fmaf(v[e], fmaf(v[e], k3, k2), k1), e0);
    store8<T>(o + i, v);
  }
}

extern "C" int odi_poly_norm(const void* z, const float* coef, void* out, int rows, int F, float eps, int dtype,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (F <= 0) return ODI_ERR_ARGUMENT;
  const int threads = F >= 2048 ? 256 : 128;
  if (F % 8 == 0 && (((uintptr_t)z | (uintptr_t)out) & 15) == 0) {
    if (dtype == 0) odi_rc = launch_pdl((poly_norm_vec_kernel<float>), dim3(rows), dim3(threads), 0, stream, (const float*)z, coef, (float*)out, F, eps);
    else odi_rc = launch_pdl((poly_norm_vec_kernel<bf16>), dim3(rows), dim3(threads), 0, stream, (const bf16*)z, coef, (bf16*)out, F, eps);
    return launch_status();
  }
  if (dtype == 0) odi_rc = launch_pdl((poly_norm_kernel<float>), dim3(rows), dim3(threads), 0, stream, (const float*)z, coef, (float*)out, F, eps);
  else odi_rc = launch_pdl((poly_norm_kernel<bf16>), dim3(rows), dim3(threads), 0, stream, (const bf16*)z, coef, (bf16*)out, F, eps);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// x += m y (fp32, in place)
// ---------------------------------------------------------------------------------
__global__ void scaled_add_kernel(float* __restrict__ x, const float* __restrict__ y, long n, float m) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
    float4 xv = *(float4*)(x + i);
    const float4 yv = *(const float4*)(y + i);
    xv.x = fmaf(m, yv.x, xv.x); xv.y = fmaf(m, yv.y, xv.y); xv.z = fmaf(m, yv.z, xv.z); xv.w = fmaf(m, yv.w, xv.w);
    *(float4*)(x + i) = xv;
  } else {
    for (long j = i; j < n && j < i + 4; ++j) x[j] = fmaf(m, y[j], x[j]);
  }
}

extern "C" int odi_scaled_add(float* x, const float* y, long n, float m, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long blocks = (n + 1023) / 1024;
  if (blocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
  odi_rc = launch_pdl((scaled_add_kernel), dim3((unsigned)blocks), dim3(256), 0, stream, x, y, n, m);
  return launch_status();
}
