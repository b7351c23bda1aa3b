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
//              a column lives in the registers of 8 or 16 lanes, the read-out is a sum over those lanes; 16 tokens of B, C, x
//              and the decays are staged in shared memory at a time, the next 16 by asynchronous copies meanwhile.
//  gate_norm   v = y * silu(z); v is RMS-normed in `norm_groups` equal parts of a token's row (each part by its own
//              root mean square, eps inside the root), times a weight per lane, rounded once to T.
//
// Everything but the projection's own output is fp32 in both compute dtypes.
#include "common.cuh"
#include <type_traits>

#define SSD_MAX_TAPS 16
#define SSD_TCH 16          // tokens staged at a time
#define SSD_COLS 32         // most columns of S per block (a kernel form takes 32 or 8)

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

__device__ __forceinline__ void ssd_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ssd_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ssd_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ssd_cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// LANES: lanes that share a column of S (8 or 16); NPT: rows of S per lane (N <= LANES NPT).  VEC (N a multiple of 4,
// 16-byte aligned rows of xbc): a lane owns rows 4 (ns + LANES j) .. + 3 of its column and reads B and C four at a time;
// else rows ns + LANES k, one at a time.
// Two staging buffers: while the block works through one chunk of SSD_TCH tokens, the asynchronous copies of the next
// chunk's B, C and x (and the loads of its step sizes) are in flight; one barrier per chunk.
// COLS: columns of S per block (COLS * 8 threads): fewer columns make more blocks, which is what a step of one long
// sequence needs, since each warp's time is the chain of its tokens.
template <typename T, int NPT, bool VEC, int COLS, int LANES>
__global__ void __launch_bounds__(COLS * LANES)
ssd_scan_kernel(SsdArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float ssd_smem[];
  const int N = a.N, P = a.P, inner = a.heads * P, C = inner + 2 * a.G * N;
  const int stage = SSD_TCH * (2 * N + COLS) + 2 * SSD_TCH;      // floats of one buffer
  const int tid = threadIdx.x, ns = tid % LANES, pc = tid / LANES;
  const int h = blockIdx.y, seq = blockIdx.z, g = h / (a.heads / a.G);
  const int p0 = blockIdx.x * COLS, p = p0 + pc;
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  if (q_len <= 0) return;
  const int slot = a.slots[seq];
  float* S = a.state + ((size_t)slot * a.heads + h) * N * P;
  auto row_of = [&](int k) { return VEC ? 4 * (ns + LANES * (k >> 2)) + (k & 3) : ns + LANES * k; };
  float s[NPT];
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int n = row_of(k);
    s[k] = (n < N && p < P) ? S[(size_t)n * P + p] : 0.f;
  }
  const float neg_a = -expf(a.a_log[h]), dt_b = a.dt_bias[h], dskip = a.d_skip[h];
  const T* dt_col = (const T*)a.proj + 2 * inner + 2 * a.G * N + h;
  const int n_chunks = (q_len + SSD_TCH - 1) / SSD_TCH;

  // buffer layout: B [TCH][N], C [TCH][N], x [TCH][COLS], dt [TCH], decay [TCH]
  auto issue = [&](int c) {
    float* buf = ssd_smem + (size_t)(c & 1) * stage;
    const int base = c * SSD_TCH, nt = min(SSD_TCH, q_len - base);
    const float* rows = a.xbc + (size_t)(q_begin + base) * C;
    // a warp copies a token's B and C rows, token after token (no division in the loop)
    const int warp = tid >> 5, lane = tid & 31, n_warps = (COLS * LANES) >> 5;
    for (int tt = warp; tt < nt; tt += n_warps) {
      const float* src = rows + (size_t)tt * C + inner + (size_t)g * N;
      float* dB = buf + tt * N;
      float* dC = buf + SSD_TCH * N + tt * N;
      if (VEC) {
        for (int j = 4 * lane; j < N; j += 128) { ssd_cp16(dB + j, src + j); ssd_cp16(dC + j, src + (size_t)a.G * N + j); }
      } else {
        for (int n = lane; n < N; n += 32) { ssd_cp4(dB + n, src + n); ssd_cp4(dC + n, src + (size_t)a.G * N + n); }
      }
    }
    float* sX = buf + 2 * SSD_TCH * N;
    for (int i = tid; i < nt * COLS; i += blockDim.x) {
      const int tt = i / COLS, cc = i % COLS;
      if (p0 + cc < P) ssd_cp4(sX + i, rows + (size_t)tt * C + (size_t)h * P + p0 + cc);
      else sX[i] = 0.f;
    }
    ssd_cp_commit();
  };
  auto step_sizes = [&](int c, float raw) {      // by thread tid < tokens of chunk c
    float* buf = ssd_smem + (size_t)(c & 1) * stage + SSD_TCH * (2 * N + COLS);
    const float dt = ssd_softplus(raw + dt_b);
    buf[tid] = dt;
    buf[SSD_TCH + tid] = expf(neg_a * dt);
  };

  issue(0);
  if (tid < min(SSD_TCH, q_len)) step_sizes(0, to_f<T>(dt_col[(size_t)(q_begin + tid) * a.ld]));
  for (int c = 0; c < n_chunks; ++c) {
    ssd_cp_wait_all();
    __syncthreads();      // chunk c is in its buffer; everybody has left chunk c - 1, whose buffer takes chunk c + 1
    const int base = c * SSD_TCH, nt = min(SSD_TCH, q_len - base);
    const bool more = c + 1 < n_chunks;
    const int nt_next = more ? min(SSD_TCH, q_len - base - SSD_TCH) : 0;
    float raw_next = 0.f;
    if (more) {
      issue(c + 1);
      if (tid < nt_next) raw_next = to_f<T>(dt_col[(size_t)(q_begin + base + SSD_TCH + tid) * a.ld]);
    }
    const float* buf = ssd_smem + (size_t)(c & 1) * stage;
    const float* sB = buf;
    const float* sC = buf + SSD_TCH * N;
    const float* sX = buf + 2 * SSD_TCH * N;
    const float* sDt = sX + SSD_TCH * COLS;
    const float* sDa = sDt + SSD_TCH;
    // one token: the state's rows of this lane move on, the read-out is summed over the column's lanes
    auto token = [&](int tt, auto full_tag) {
      constexpr bool FULL = decltype(full_tag)::value;      // N == 8 NPT: no row of the lane lies beyond the state
      const float x = sX[tt * COLS + pc], dt = sDt[tt], da = sDa[tt];
      const float dx = dt * x;
      const float* B = sB + tt * N;
      const float* Cc = sC + tt * N;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (VEC) {
#pragma unroll
        for (int j = 0; j < NPT / 4; ++j) {
          const int n = 4 * (ns + LANES * j);
          if (FULL || n < N) {
            const float4 b = *(const float4*)(B + n), cv = *(const float4*)(Cc + n);
            s[4 * j] = fmaf(da, s[4 * j], dx * b.x);         acc[0] = fmaf(s[4 * j], cv.x, acc[0]);
            s[4 * j + 1] = fmaf(da, s[4 * j + 1], dx * b.y); acc[1] = fmaf(s[4 * j + 1], cv.y, acc[1]);
            s[4 * j + 2] = fmaf(da, s[4 * j + 2], dx * b.z); acc[2] = fmaf(s[4 * j + 2], cv.z, acc[2]);
            s[4 * j + 3] = fmaf(da, s[4 * j + 3], dx * b.w); acc[3] = fmaf(s[4 * j + 3], cv.w, acc[3]);
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < NPT; ++k) {
          const int n = ns + LANES * k;
          if (FULL || n < N) {
            s[k] = fmaf(da, s[k], dx * B[n]);
            acc[k & 3] = fmaf(s[k], Cc[n], acc[k & 3]);
          }
        }
      }
      float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (ns == 0 && p < P) a.y[(size_t)(q_begin + base + tt) * inner + (size_t)h * P + p] = fmaf(dskip, x, sum);
    };
    // four tokens at a time: the state goes through them in order, their four read-outs are summed over the column's
    // lanes side by side, so that the shuffles' latency is paid once per four tokens (full states, VEC form)
    auto tokens4 = [&](int t0) {
      float x[4], dx[4], da[4], acc[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        x[u] = sX[(t0 + u) * COLS + pc];
        dx[u] = sDt[t0 + u] * x[u];
        da[u] = sDa[t0 + u];
        acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < NPT / 4; ++j) {
        const int n = 4 * (ns + LANES * j);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float4 b = *(const float4*)(sB + (t0 + u) * N + n), cv = *(const float4*)(sC + (t0 + u) * N + n);
          s[4 * j] = fmaf(da[u], s[4 * j], dx[u] * b.x);         acc[u][0] = fmaf(s[4 * j], cv.x, acc[u][0]);
          s[4 * j + 1] = fmaf(da[u], s[4 * j + 1], dx[u] * b.y); acc[u][1] = fmaf(s[4 * j + 1], cv.y, acc[u][1]);
          s[4 * j + 2] = fmaf(da[u], s[4 * j + 2], dx[u] * b.z); acc[u][2] = fmaf(s[4 * j + 2], cv.z, acc[u][2]);
          s[4 * j + 3] = fmaf(da[u], s[4 * j + 3], dx[u] * b.w); acc[u][3] = fmaf(s[4 * j + 3], cv.w, acc[u][3]);
        }
      }
      float sum[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) sum[u] = (acc[u][0] + acc[u][1]) + (acc[u][2] + acc[u][3]);
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], o);
      }
      if (ns == 0 && p < P) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
          a.y[(size_t)(q_begin + base + t0 + u) * inner + (size_t)h * P + p] = fmaf(dskip, x[u], sum[u]);
      }
    };
    if (N == LANES * NPT) {
      int tt = 0;
      if (VEC) {
        for (; tt + 4 <= nt; tt += 4) tokens4(tt);
      }
      for (; tt < nt; ++tt) token(tt, std::true_type{});
    } else {
      for (int tt = 0; tt < nt; ++tt) token(tt, std::false_type{});
    }
    if (more && tid < nt_next) step_sizes(c + 1, raw_next);
  }
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int n = row_of(k);
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
  // Two forms: 32 columns a block when that already gives two blocks per multiprocessor (many sequences); else 8
  // columns, four times the blocks, since a warp's time is the chain of its sequence's tokens and a step of one long
  // sequence has nothing else to run beside it.  (Measured at 32 heads of 64 columns, 128 rows, 2,048 tokens: 32
  // columns 1,080 us, 8 columns 545 us, 8 columns over 16 lanes each 640 us.)
  const bool narrow = (long)((a.P + 31) / 32) * a.heads * a.n_seqs < 2 * 148;
  const int cols = narrow ? 8 : SSD_COLS;
  const dim3 grid((a.P + cols - 1) / cols, a.heads, a.n_seqs);
  const size_t smem = 2 * sizeof(float) * (SSD_TCH * (2 * (size_t)a.N + cols) + 2 * SSD_TCH);
  const int C_all = a.heads * a.P + 2 * a.G * a.N;
  const bool vec = a.N % 4 == 0 && C_all % 4 == 0 && (a.heads * a.P) % 4 == 0 && ((uintptr_t)a.xbc & 15) == 0;
  if (odi_rc == 0) {
#define ODI_SCAN_FORM(NPT, VEC, COLS, LANES) \
    do { if (smem > 48 * 1024) { \
           const cudaError_t e = cudaFuncSetAttribute(ssd_scan_kernel<T, NPT, VEC, COLS, LANES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
           if (e != cudaSuccess) return (int)e; } \
         odi_rc = launch_pdl((ssd_scan_kernel<T, NPT, VEC, COLS, LANES>), grid, dim3(COLS * LANES), smem, stream, a); } while (0)
#define ODI_SCAN(NPT_WIDE, NPT_NARROW) \
    do { if (vec) { if (narrow) ODI_SCAN_FORM(NPT_NARROW, true, 8, 8); else ODI_SCAN_FORM(NPT_WIDE, true, 32, 8); } \
         else { if (narrow) ODI_SCAN_FORM(NPT_NARROW, false, 8, 8); else ODI_SCAN_FORM(NPT_WIDE, false, 32, 8); } } while (0)
    if (a.N <= 32) ODI_SCAN(4, 4); else if (a.N <= 64) ODI_SCAN(8, 8); else if (a.N <= 128) ODI_SCAN(16, 16); else ODI_SCAN(32, 32);
#undef ODI_SCAN
#undef ODI_SCAN_FORM
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
