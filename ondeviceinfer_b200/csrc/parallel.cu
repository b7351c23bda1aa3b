// Kernels of a block whose mixer and feed-forward read ONE norm of the stream side by side,
//   h = norm(x);  x <- x + m (mixer(h + conv(h)) + ff(h)),
// with a short causal convolution over time in front of the mixer, and of a feed-forward whose activation is a
// polynomial of row-normed powers:
//
//  * canon_norm: per token the norm of its row (one number g as the weight), h in T for the feed-forward, and
//    h + conv(h) in T for the mixer, conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j).  The rows before t come from
//    the step's own tokens (their norm is taken again: the rows are in L2) or, before the first token that a
//    sequence brings, from the sequence's state: h of its last taps - 1 positions, fp32, zero before its start.
//  * canon_state: afterwards, the state of every sequence moved on by the tokens it brought.
//  * poly_norm: out = a N(z) + b N(z^2) + c N(z^3) + e, N(v) = v / sqrt(mean(v^2) + eps) over a token's row.
//  * scaled_add: x += m y on fp32 rows.
// Norms, the convolution's sum and the powers are fp32 in both compute dtypes; each output is rounded once.
#include "common.cuh"

#define CANON_MAX_TAPS 8

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
  const int t = blockIdx.x;
  const int seq = a.tok_seq[t];
  const int i = t - a.cu_q[seq];            // index among the tokens that the sequence brings in this step
  const int W = a.W, taps = a.taps;
  const float g = a.g[0];
  float inv[CANON_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < CANON_MAX_TAPS; ++k) {
    inv[k] = 0.f;
    if (k < taps && i - k >= 0) {
      const float* xr = a.x + (size_t)(t - k) * W;
      float ss = 0.f;
      for (int c = threadIdx.x; c < W; c += blockDim.x) { const float v = xr[c]; ss += v * v; }
      ss = block_sum(ss, scratch);
      inv[k] = g / sqrtf(ss / (float)W + a.eps);
    }
  }
  const float* st = a.state != nullptr ? a.state + (size_t)a.slots[seq] * (taps - 1) * W : nullptr;
  T* h = (T*)a.h_out + (size_t)t * W;
  T* hc = (T*)a.hc_out + (size_t)t * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float h0 = a.x[(size_t)t * W + c] * inv[0];
    const float* w = a.taps_w + (size_t)c * taps;
    float acc = h0 * w[taps - 1];
#pragma unroll
    for (int k = 1; k < CANON_MAX_TAPS; ++k) {
      if (k < taps) {
        // position t - k: a token of this step, or row (taps - 1) + (i - k) of the state
        const float hk = i - k >= 0 ? a.x[(size_t)(t - k) * W + c] * inv[k] : st[(size_t)(taps - 1 + i - k) * W + c];
        acc = fmaf(hk, w[taps - 1 - k], acc);
      }
    }
    h[c] = from_f<T>(h0);
    hc[c] = from_f<T>(h0 + acc);
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

extern "C" int odi_canon_norm(const CanonArgs* args, int dtype, cudaStream_t stream) {
  const CanonArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (a.taps < 1 || a.taps > CANON_MAX_TAPS || a.W <= 0 || (a.taps > 1 && a.state == nullptr)) return ODI_ERR_UNSUPPORTED;
  const int threads = a.W >= 1024 ? 256 : 128;
  if (dtype == 0) odi_rc = launch_pdl((canon_norm_kernel<float>), dim3(a.n_tokens), dim3(threads), 0, stream, a);
  else odi_rc = launch_pdl((canon_norm_kernel<bf16>), dim3(a.n_tokens), dim3(threads), 0, stream, a);
  return launch_status();
}

extern "C" int odi_canon_state(const CanonArgs* args, cudaStream_t stream) {
  const CanonArgs a = *args;
  if (a.n_seqs <= 0 || a.taps <= 1) return 0;
  if (a.taps > CANON_MAX_TAPS || a.state == nullptr) return ODI_ERR_UNSUPPORTED;
  odi_rc = launch_pdl((canon_state_kernel), dim3(a.n_seqs), dim3(a.W >= 1024 ? 256 : 128), 0, stream, a);
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

extern "C" int odi_poly_norm(const void* z, const float* coef, void* out, int rows, int F, float eps, int dtype,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (F <= 0) return ODI_ERR_ARGUMENT;
  const int threads = F >= 2048 ? 256 : 128;
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
