// A selective state-space mixer with a scalar decay per head (the recurrent form of the state-space duality):
// what lies between its input projection and its output projection.
//
// A token's row of the input projection is [ z: inner | x: inner | B: G N | C: G N | dt: heads ], inner = heads P.
//
//  conv        x, B and C together (inner + 2 G N channels) pass a causal convolution over time per channel,
//              taps w[c, 0..taps-1] (the last one is the current token's) and a bias, then SiLU; inputs before the
//              first token that a sequence brings come from its state (its last taps - 1 inputs, fp32, zero before
//              its start).  fp32 sums; the result stays fp32 for the recurrence.
//  conv_state  the state moved on by the tokens that the sequence brought.
//  scan        per sequence and head h (group g = h / (heads / G)), over the sequence's tokens in order:
//                dt = softplus(dt_raw + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt B_g x_h^T;  y = S^T C_g + D[h] x_h
//              with S [N, P] fp32 per (sequence, head), kept in the cache between steps.  A block owns 32 columns of S;
//              a column lives in the registers of 8 lanes (every 8th row each), the read-out is a sum over those
//              lanes; 16 tokens of B, C, x and the decays are staged in shared memory at a time.
//  gate_norm   v = y * silu(z); v is RMS-normed in `norm_groups` equal parts of a token's row (each part by its own
//              root mean square, eps inside the root), times a weight per lane, rounded once to T.
//
// Everything but the projection's own output is fp32 in both compute dtypes.
#include "common.cuh"

#define SSD_MAX_TAPS 16
#define SSD_TCH 16          // tokens staged at a time
#define SSD_COLS 32         // columns of S per block
#define SSD_LANES 8         // lanes that share a column

struct SsdArgs {
  const void* proj;       // [n_tokens, ld] in T
  const float* conv_w;    // [C, taps]
  const float* conv_b;    // [C]
  const float* dt_bias;   // [heads]
  const float* a_log;     // [heads]
  const float* d_skip;    // [heads]
  const float* norm_w;    // [inner]
  float* conv_state;      // [slots, taps - 1, C]; null when taps == 1
  float* state;           // [slots, heads, N, P]
  float* xbc;             // [n_tokens, C] scratch
  float* y;               // [n_tokens, inner] scratch
  void* out;              // [n_tokens, inner] in T
  const int* cu_q;        // [n_seqs + 1]
  const int* tok_seq;     // [n_tokens]
  const int* slots;       // [n_seqs]
  int n_tokens, n_seqs, ld, heads, P, N, G, taps, norm_groups;
  float eps;
};

__device__ __forceinline__ float ssd_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float ssd_silu(float x) { return x / (1.f + expf(-x)); }

template <typename T>
__device__ __forceinline__ float ssd_conv_input(const SsdArgs& a, int inner, int C, int q_begin, int slot, int idx, int c) {
  // input `idx` of the sequence's run in this step; negative indices reach into the convolution state
  if (idx >= 0) return to_f<T>(((const T*)a.proj)[(size_t)(q_begin + idx) * a.ld + inner + c]);
  return a.conv_state[((size_t)slot * (a.taps - 1) + (a.taps - 1 + idx)) * C + c];
}

template <typename T>
__global__ void __launch_bounds__(256)
ssd_conv_kernel(SsdArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int inner = a.heads * a.P, C = inner + 2 * a.G * a.N;
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int seq = a.tok_seq[t];
  const int q_begin = a.cu_q[seq], slot = a.slots[seq];
  const int li = t - q_begin;
  float acc = a.conv_b[c];
  for (int j = 0; j < a.taps; ++j)
    acc = fmaf(a.conv_w[(size_t)c * a.taps + j], ssd_conv_input<T>(a, inner, C, q_begin, slot, li - (a.taps - 1) + j, c), acc);
  a.xbc[(size_t)t * C + c] = ssd_silu(acc);
}

template <typename T>
__global__ void __launch_bounds__(256)
ssd_conv_state_kernel(SsdArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int inner = a.heads * a.P, C = inner + 2 * a.G * a.N;
  const int seq = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin, slot = a.slots[seq];
  const int keep = a.taps - 1;
  float next[SSD_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SSD_MAX_TAPS; ++j)
    if (j < keep) next[j] = ssd_conv_input<T>(a, inner, C, q_begin, slot, q_len - keep + j, c);
#pragma unroll
  for (int j = 0; j < SSD_MAX_TAPS; ++j)
    if (j < keep) a.conv_state[((size_t)slot * keep + j) * C + c] = next[j];
}

// NPT: rows of S per lane (N <= 8 NPT).
template <typename T, int NPT>
__global__ void __launch_bounds__(SSD_COLS * SSD_LANES)
ssd_scan_kernel(SsdArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float ssd_smem[];
  const int N = a.N, P = a.P, inner = a.heads * P, C = inner + 2 * a.G * N;
  float* sB = ssd_smem;                       // [TCH][N]
  float* sC = sB + SSD_TCH * N;               // [TCH][N]
  float* sX = sC + SSD_TCH * N;               // [TCH][COLS]
  float* sDt = sX + SSD_TCH * SSD_COLS;       // [TCH]
  float* sDa = sDt + SSD_TCH;                 // [TCH]
  const int tid = threadIdx.x, ns = tid % SSD_LANES, pc = tid / SSD_LANES;
  const int h = blockIdx.y, seq = blockIdx.z, g = h / (a.heads / a.G);
  const int p0 = blockIdx.x * SSD_COLS, p = p0 + pc;
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  if (q_len <= 0) return;
  const int slot = a.slots[seq];
  float* S = a.state + ((size_t)slot * a.heads + h) * N * P;
  float s[NPT];
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int n = ns + SSD_LANES * k;
    s[k] = (n < N && p < P) ? S[(size_t)n * P + p] : 0.f;
  }
  const float neg_a = -expf(a.a_log[h]), dt_b = a.dt_bias[h], dskip = a.d_skip[h];
  const T* proj = (const T*)a.proj;
  for (int base = 0; base < q_len; base += SSD_TCH) {
    const int nt = min(SSD_TCH, q_len - base);
    __syncthreads();      // the chunk before has been consumed
    for (int i = tid; i < nt * N; i += blockDim.x) {
      const int tt = i / N, n = i % N;
      const float* row = a.xbc + (size_t)(q_begin + base + tt) * C + inner + (size_t)g * N;
      sB[tt * N + n] = row[n];
      sC[tt * N + n] = row[(size_t)a.G * N + n];
    }
    for (int i = tid; i < nt * SSD_COLS; i += blockDim.x) {
      const int tt = i / SSD_COLS, cc = i % SSD_COLS;
      sX[i] = p0 + cc < P ? a.xbc[(size_t)(q_begin + base + tt) * C + (size_t)h * P + p0 + cc] : 0.f;
    }
    if (tid < nt) {
      const float raw = to_f<T>(proj[(size_t)(q_begin + base + tid) * a.ld + 2 * inner + 2 * a.G * N + h]);
      const float dt = ssd_softplus(raw + dt_b);
      sDt[tid] = dt;
      sDa[tid] = expf(neg_a * dt);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float x = sX[tt * SSD_COLS + pc], dt = sDt[tt], da = sDa[tt];
      const float dx = dt * x;
      const float* B = sB + tt * N;
      const float* Cc = sC + tt * N;
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < NPT; ++k) {
        const int n = ns + SSD_LANES * k;
        if (n < N) {
          s[k] = fmaf(da, s[k], dx * B[n]);
          acc = fmaf(s[k], Cc[n], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (ns == 0 && p < P) a.y[(size_t)(q_begin + base + tt) * inner + (size_t)h * P + p] = fmaf(dskip, x, acc);
    }
  }
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int n = ns + SSD_LANES * k;
    if (n < N && p < P) S[(size_t)n * P + p] = s[k];
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
ssd_gate_norm_kernel(SsdArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int inner = a.heads * a.P, part = inner / a.norm_groups;
  const int t = blockIdx.x, grp = blockIdx.y;
  const T* z = (const T*)a.proj + (size_t)t * a.ld + (size_t)grp * part;
  const float* y = a.y + (size_t)t * inner + (size_t)grp * part;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float v = y[i] * ssd_silu(to_f<T>(z[i]));
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)part + a.eps);
  T* out = (T*)a.out + (size_t)t * inner + (size_t)grp * part;
  const float* w = a.norm_w + (size_t)grp * part;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float v = y[i] * ssd_silu(to_f<T>(z[i]));
    out[i] = from_f<T>(v * inv * w[i]);
  }
}

template <typename T>
static int ssd_launch(const SsdArgs& a, cudaStream_t stream) {
  const int inner = a.heads * a.P, C = inner + 2 * a.G * a.N;
  odi_rc = launch_pdl((ssd_conv_kernel<T>), dim3(a.n_tokens, (C + 255) / 256), dim3(256), 0, stream, a);
  if (odi_rc == 0 && a.taps > 1)
    odi_rc = launch_pdl((ssd_conv_state_kernel<T>), dim3(a.n_seqs, (C + 255) / 256), dim3(256), 0, stream, a);
  const dim3 grid((a.P + SSD_COLS - 1) / SSD_COLS, a.heads, a.n_seqs);
  const size_t smem = sizeof(float) * (SSD_TCH * (2 * (size_t)a.N + SSD_COLS) + 2 * SSD_TCH);
  if (odi_rc == 0) {
#define ODI_SCAN(NPT) odi_rc = launch_pdl((ssd_scan_kernel<T, NPT>), grid, dim3(SSD_COLS * SSD_LANES), smem, stream, a)
    if (a.N <= 32) ODI_SCAN(4); else if (a.N <= 64) ODI_SCAN(8); else if (a.N <= 128) ODI_SCAN(16); else ODI_SCAN(32);
#undef ODI_SCAN
  }
  if (odi_rc == 0)
    odi_rc = launch_pdl((ssd_gate_norm_kernel<T>), dim3(a.n_tokens, a.norm_groups), dim3(256), 0, stream, a);
  return launch_status();
}

// Kernels launched by one call: 3, or 4 with a convolution state.
extern "C" int odi_ssd(const SsdArgs* args, int dtype, cudaStream_t stream) {
  const SsdArgs a = *args;
  if (a.n_tokens <= 0 || a.n_seqs <= 0) return 0;
  if (a.heads <= 0 || a.P <= 0 || a.N <= 0 || a.G <= 0 || a.heads % a.G != 0 || a.taps < 1 || a.norm_groups <= 0 ||
      (a.heads * a.P) % a.norm_groups != 0)
    return ODI_ERR_ARGUMENT;
  if (a.N > 256 || a.taps > SSD_MAX_TAPS || a.heads > 65535 || a.n_seqs > 65535 || a.norm_groups > 65535) return ODI_ERR_UNSUPPORTED;
  if (a.taps > 1 && a.conv_state == nullptr) return ODI_ERR_ARGUMENT;
  return dtype == 0 ? ssd_launch<float>(a, stream) : ssd_launch<bf16>(a, stream);
}
