// Kernels around an attention whose queries and keys are rotated and then scaled to unit root mean square, and
// around blocks that norm a sublayer's output before adding it:
//
//  * rot_unit_prep: per (token, head) the rotation of neighbouring-lane pairs over the first rot_dim lanes, the
//    division by sqrt(mean of squares + eps), optionally times a weight per lane (one for all query heads, one for
//    all key heads), and the write of q to the query buffer, k and v to their cache pages (v has a width of its own);
//  * activation: out = act(x), act the exact (erf) GELU, its tanh form or the square of max(x, 0), fp32 arithmetic,
//    one rounding;
//  * softcap: x <- c tanh(x / c) in place on fp32 rows (logits);
//  * concat_cast: out[t] = [a[t] ; b[t]] of two fp32 streams in the compute dtype;
//  * rmsnorm_add: h[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w, all fp32 (the norm after a sublayer and the
//    residual add in one pass);
//  * rmsnorm_add_norm: the same followed by the norm that the next sublayer takes of the sum, the row kept in registers;
//  * gated_row_add: acc[t] += sigmoid(x[t] . g) * y[t] (an expert that every token takes, scaled by a number per token).
#include "common.cuh"

struct RotUnitArgs {
  const void* qkv;      // [n_tokens, nq * d + nkv * d + nkv * dv]
  void* q_out;          // [n_tokens, nq * d_store]
  void* k_pool;         // [pages, nkv, page_size, d_store]
  void* v_pool;         // [pages, nkv, page_size, dv]
  const float* cos_t;   // null: no rotation; [n_tokens, rot_dim / 2]
  const float* sin_t;
  const int* tok_seq;
  const int* tok_pos;
  const int* page_start;
  const int* page_ids;
  int n_tokens, nq, nkv, d, dv, rot_dim, page_size, ring_pages, write_kv, unit;
  int d_store;          // lanes of a stored q or k head, >= d; the lanes beyond d are written as zero
  float eps;
  int v_from_k;         // 1: there are no v lanes in `qkv`; the value of a head is its key as projected, before the rotation (dv == d)
  const float* q_w;     // null, or [d]: after the division every query head is multiplied by it lane by lane
  const float* k_w;     // the same for the key heads
};

// One warp per (token, head).  Lane i % 32 holds element i in register i / 32, so the partner of lane 2i
// (lane 2i + 1) is the neighbouring lane of the same register.
template <typename T, int MAXP>
__global__ void rot_unit_prep_kernel(RotUnitArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = a.nq + (a.write_kv ? 2 * a.nkv : 0);
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)a.n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int d = a.d;
  const size_t row = (size_t)(a.nq + a.nkv) * d + (a.v_from_k ? (size_t)0 : (size_t)a.nkv * a.dv);
  const int kind = h < a.nq ? 0 : (h < a.nq + a.nkv ? 1 : 2);  // 0 q, 1 k, 2 v
  const int pos = a.tok_pos[t];
  const T* src;
  T* dst;
  if (kind == 0) {
    src = (const T*)a.qkv + (size_t)t * row + (size_t)h * d;
    dst = (T*)a.q_out + ((size_t)t * a.nq + h) * a.d_store;
  } else {
    const int hk = kind == 1 ? h - a.nq : h - a.nq - a.nkv;
    const int s = a.tok_seq[t];
    const int page = a.page_ids[a.page_start[s] + page_slot_of(pos, a.page_size, a.ring_pages)];
    const size_t at = ((size_t)page * a.nkv + hk) * a.page_size + (pos % a.page_size);
    if (kind == 1) {
      src = (const T*)a.qkv + (size_t)t * row + (size_t)(a.nq + hk) * d;
      dst = (T*)a.k_pool + at * a.d_store;
    } else {
      src = a.v_from_k ? (const T*)a.qkv + (size_t)t * row + (size_t)(a.nq + hk) * d
                       : (const T*)a.qkv + (size_t)t * row + (size_t)(a.nq + a.nkv) * d + (size_t)hk * a.dv;
      dst = (T*)a.v_pool + at * a.dv;
      for (int i = lane; i < a.dv; i += 32) dst[i] = src[i];
      return;
    }
  }
  float x[MAXP];
#pragma unroll
  for (int r = 0; r < MAXP; ++r) {
    const int i = lane + 32 * r;
    x[r] = i < d ? to_f<T>(src[i]) : 0.f;
  }
  if (a.cos_t != nullptr) {
    const int half = a.rot_dim >> 1;
#pragma unroll
    for (int r = 0; r < MAXP; ++r) {
      const int i = lane + 32 * r;
      const float other = __shfl_xor_sync(0xffffffffu, x[r], 1);
      if (i < a.rot_dim) {
        const float cs = a.cos_t[(size_t)t * half + (i >> 1)], sn = a.sin_t[(size_t)t * half + (i >> 1)];
        // even lane u: u cos - v sin; odd lane v: v cos + u sin
        x[r] = (i & 1) ? fmaf(other, sn, x[r] * cs) : fmaf(-other, sn, x[r] * cs);
      }
    }
  }
  if (a.unit) {
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < MAXP; ++r) ss += x[r] * x[r];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + a.eps);
    const float* w = kind == 0 ? a.q_w : a.k_w;
#pragma unroll
    for (int r = 0; r < MAXP; ++r) {
      const int i = lane + 32 * r;
      x[r] *= (w != nullptr && i < d) ? inv * w[i] : inv;
    }
  }
#pragma unroll
  for (int r = 0; r < MAXP; ++r) {
    const int i = lane + 32 * r;
    if (i < a.d_store) dst[i] = from_f<T>(i < d ? x[r] : 0.f);
  }
}

// bf16 heads whose width is a multiple of 4 (d == d_store): a lane holds four neighbouring lanes of the head per
// step of 128, so both members of a rotated pair sit in one thread, and every access is 8 bytes wide.  A warp
// takes `heads_per_warp` heads of one token one after the other.  Same arithmetic as rot_unit_prep_kernel.
template <int MAXP4>
__global__ void rot_unit_prep_vec_kernel(RotUnitArgs a, int heads_per_warp) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = a.nq + (a.write_kv ? 2 * a.nkv : 0);
  const int groups = (heads + heads_per_warp - 1) / heads_per_warp;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)a.n_tokens * groups) return;
  const int t = (int)(item / groups), h_begin = (int)(item % groups) * heads_per_warp;
  const int d = a.d, half = a.rot_dim >> 1;
  const size_t row = (size_t)(a.nq + a.nkv) * d + (a.v_from_k ? (size_t)0 : (size_t)a.nkv * a.dv);
  const bf16* base = (const bf16*)a.qkv + (size_t)t * row;
  const int pos = a.tok_pos[t];
  size_t at = 0;
  if (a.write_kv) {
    const int s = a.tok_seq[t];
    const int page = a.page_ids[a.page_start[s] + page_slot_of(pos, a.page_size, a.ring_pages)];
    at = (size_t)page * a.nkv * a.page_size + (pos % a.page_size);
  }
  for (int h = h_begin; h < min(heads, h_begin + heads_per_warp); ++h) {
    const int kind = h < a.nq ? 0 : (h < a.nq + a.nkv ? 1 : 2);
    if (kind == 2) {
      const int hk = h - a.nq - a.nkv;
      const bf16* src = a.v_from_k ? base + (size_t)(a.nq + hk) * d : base + (size_t)(a.nq + a.nkv) * d + (size_t)hk * a.dv;
      bf16* dst = (bf16*)a.v_pool + (at + (size_t)hk * a.page_size) * a.dv;
      for (int i = lane; i < a.dv; i += 32) dst[i] = src[i];
      continue;
    }
    const int hk = h - a.nq;
    const bf16* src = base + (size_t)h * d;         // q heads, then k heads, follow one another in the row
    bf16* dst = kind == 0 ? (bf16*)a.q_out + ((size_t)t * a.nq + h) * d
                          : (bf16*)a.k_pool + (at + (size_t)hk * a.page_size) * d;
    float x[MAXP4][4];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < MAXP4; ++r) {
      const int i = 4 * lane + 128 * r;
      if (i < d) {
        const uint2 raw = *(const uint2*)(src + i);
        const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x), hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
        x[r][0] = lo.x; x[r][1] = lo.y; x[r][2] = hi.x; x[r][3] = hi.y;
        if (a.cos_t != nullptr && i < a.rot_dim) {
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            if (i + 2 * pr < a.rot_dim) {
              const float cs = a.cos_t[(size_t)t * half + (i >> 1) + pr], sn = a.sin_t[(size_t)t * half + (i >> 1) + pr];
              const float u = x[r][2 * pr], v = x[r][2 * pr + 1];
              x[r][2 * pr] = fmaf(-v, sn, u * cs);
              x[r][2 * pr + 1] = fmaf(u, sn, v * cs);
            }
          }
        }
        ss += x[r][0] * x[r][0] + x[r][1] * x[r][1] + x[r][2] * x[r][2] + x[r][3] * x[r][3];
      } else {
        x[r][0] = x[r][1] = x[r][2] = x[r][3] = 0.f;
      }
    }
    float inv = 1.f;
    const float* w = nullptr;
    if (a.unit) {
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)d + a.eps);
      w = kind == 0 ? a.q_w : a.k_w;
    }
#pragma unroll
    for (int r = 0; r < MAXP4; ++r) {
      const int i = 4 * lane + 128 * r;
      if (i < d) {
        float4 f = make_float4(inv, inv, inv, inv);
        if (w != nullptr) { const float4 wv = *(const float4*)(w + i); f.x *= wv.x; f.y *= wv.y; f.z *= wv.z; f.w *= wv.w; }
        uint2 packed;
        *(__nv_bfloat162*)&packed.x = __floats2bfloat162_rn(x[r][0] * f.x, x[r][1] * f.y);
        *(__nv_bfloat162*)&packed.y = __floats2bfloat162_rn(x[r][2] * f.z, x[r][3] * f.w);
        *(uint2*)(dst + i) = packed;
      }
    }
  }
}

extern "C" int odi_rot_unit_prep(const RotUnitArgs* args, int dtype, cudaStream_t stream) {
  RotUnitArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (a.v_from_k && a.dv != a.d) return ODI_ERR_ARGUMENT;
  if (!a.unit && (a.q_w != nullptr || a.k_w != nullptr)) return ODI_ERR_ARGUMENT;
  if (((uintptr_t)a.q_w | (uintptr_t)a.k_w) % 16 != 0) return ODI_ERR_UNSUPPORTED;
  if (dtype == 1 && a.d == a.d_store && a.d % 4 == 0 && a.d <= 512 && a.d > 0 && a.dv > 0 && !(a.rot_dim & 1) && a.rot_dim <= a.d &&
      ((uintptr_t)a.qkv | (uintptr_t)a.q_out | (uintptr_t)a.k_pool) % 8 == 0 && (a.v_from_k || (a.nkv * a.dv) % 4 == 0)) {
    const int heads = a.nq + (a.write_kv ? 2 * a.nkv : 0);
    // few tokens: a warp per head for parallelism; many tokens: a warp takes a quarter of a token's heads
    const int hpw = a.n_tokens >= 256 ? (heads + 3) / 4 : 1;
    const long warps = (long)a.n_tokens * ((heads + hpw - 1) / hpw);
    const int vblocks = (int)((warps + 3) / 4);
    if (a.d <= 128) odi_rc = launch_pdl((rot_unit_prep_vec_kernel<1>), dim3(vblocks), dim3(128), 0, stream, a, hpw);
    else if (a.d <= 256) odi_rc = launch_pdl((rot_unit_prep_vec_kernel<2>), dim3(vblocks), dim3(128), 0, stream, a, hpw);
    else odi_rc = launch_pdl((rot_unit_prep_vec_kernel<4>), dim3(vblocks), dim3(128), 0, stream, a, hpw);
    return launch_status();
  }
  if (a.d_store > 512 || a.d <= 0 || a.d_store < a.d || a.dv <= 0 || (a.rot_dim & 1) || a.rot_dim > a.d) return ODI_ERR_UNSUPPORTED;
  const int heads = a.nq + (a.write_kv ? 2 * a.nkv : 0);
  const long items = (long)a.n_tokens * heads;
  const int blocks = (int)((items + 3) / 4);
#define ODI_LAUNCH(T, P) odi_rc = launch_pdl((rot_unit_prep_kernel<T, P>), dim3(blocks), dim3(128), 0, stream, a)
  if (dtype == 0) {
    if (a.d_store <= 128) ODI_LAUNCH(float, 4); else if (a.d_store <= 256) ODI_LAUNCH(float, 8); else ODI_LAUNCH(float, 16);
  } else {
    if (a.d_store <= 128) ODI_LAUNCH(bf16, 4); else if (a.d_store <= 256) ODI_LAUNCH(bf16, 8); else ODI_LAUNCH(bf16, 16);
  }
#undef ODI_LAUNCH
  return launch_status();
}

// ---------------------------------------------------------------------------------

__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f)); }
__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ float relu_squared(float z) { const float r = fmaxf(z, 0.f); return r * r; }
__device__ __forceinline__ float activation_of(float z, int kind) {
  return kind == 0 ? gelu_erf(z) : (kind == 1 ? gelu_tanh(z) : relu_squared(z));
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, long n, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float z = to_f<T>(x[i]);
  out[i] = from_f<T>(activation_of(z, kind));
}

// Eight bf16 per thread (16-byte loads and stores); n8 = n / 8.
__global__ void activation_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, long n8, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  uint4 raw = x[i];
  __nv_bfloat162* h = (__nv_bfloat162*)&raw;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    h[e] = __floats2bfloat162_rn(activation_of(f.x, kind), activation_of(f.y, kind));
  }
  out[i] = raw;
}

// kind: 0 the exact (erf) GELU, 1 its tanh form, 2 max(x, 0)^2
extern "C" int odi_activation(const void* x, void* out, long n, int kind, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (kind < 0 || kind > 2) return ODI_ERR_ARGUMENT;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == 1 && n % 8 == 0 && ((uintptr_t)x | (uintptr_t)out) % 16 == 0) {
    odi_rc = launch_pdl((activation_vec_kernel), dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, stream, (const uint4*)x, (uint4*)out, n / 8, kind);
    return launch_status();
  }
  if (dtype == 0) odi_rc = launch_pdl((activation_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)x, (float*)out, n, kind);
  else odi_rc = launch_pdl((activation_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)x, (bf16*)out, n, kind);
  return launch_status();
}

__global__ void softcap_kernel(float* __restrict__ x, long n, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int odi_softcap(float* x, long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return ODI_ERR_ARGUMENT;
  odi_rc = launch_pdl((softcap_kernel), dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap);
  return launch_status();
}

template <typename T>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out,
                                   long n, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long t = i / (2 * H);
  const int c = (int)(i % (2 * H));
  out[i] = from_f<T>(c < H ? a[t * H + c] : b[t * H + c - H]);
}

// Four elements per thread (H a multiple of 4, so the four come from one source); n4 = rows * 2 H / 4.
template <typename T>
__global__ void concat_cast_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b, T* __restrict__ out,
                                       long n4, int H4) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const long t = i / (2 * H4);
  const int c = (int)(i % (2 * H4));
  const float4 v = c < H4 ? a[t * H4 + c] : b[t * H4 + c - H4];
  if (sizeof(T) == 4) {
    ((float4*)out)[i] = v;
  } else {
    uint2 packed;
    *(__nv_bfloat162*)&packed.x = __floats2bfloat162_rn(v.x, v.y);
    *(__nv_bfloat162*)&packed.y = __floats2bfloat162_rn(v.z, v.w);
    ((uint2*)out)[i] = packed;
  }
}

extern "C" int odi_concat_cast(const float* a, const float* b, void* out, long rows, int H, int dtype, cudaStream_t stream) {
  const long n = rows * 2 * H;
  if (n <= 0) return 0;
  if (H % 4 == 0 && ((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) % 16 == 0) {
    const unsigned vblocks = (unsigned)((n / 4 + 255) / 256);
    if (dtype == 0) odi_rc = launch_pdl((concat_cast_vec_kernel<float>), dim3(vblocks), dim3(256), 0, stream, (const float4*)a, (const float4*)b, (float*)out, n / 4, H / 4);
    else odi_rc = launch_pdl((concat_cast_vec_kernel<bf16>), dim3(vblocks), dim3(256), 0, stream, (const float4*)a, (const float4*)b, (bf16*)out, n / 4, H / 4);
    return launch_status();
  }
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == 0) odi_rc = launch_pdl((concat_cast_kernel<float>), dim3(blocks), dim3(256), 0, stream, a, b, (float*)out, n, H);
  else odi_rc = launch_pdl((concat_cast_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, a, b, (bf16*)out, n, H);
  return launch_status();
}

// hidden[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w: one block per row, the row read twice (the second time from cache).
__global__ void rmsnorm_add_kernel(float* __restrict__ hidden, const float* __restrict__ y, const float* __restrict__ w,
                                   int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = y[base + i]; ss += v * v; }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) hidden[base + i] += y[base + i] * inv * w[i];
}

// The same with 16-byte accesses (H a multiple of 4); the row of y stays in registers between the two passes when
// NV float4 per thread cover it (NV = 0: it is read again).
template <int NV>
__global__ void rmsnorm_add_vec_kernel(float4* __restrict__ hidden, const float4* __restrict__ y, const float4* __restrict__ w,
                                       int H4, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * H4;
  float4 keep[NV > 0 ? NV : 1];
  float ss = 0.f;
  if (NV > 0) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      keep[j] = i < H4 ? y[base + i] : make_float4(0.f, 0.f, 0.f, 0.f);
      ss += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
    }
  } else {
    for (int i = threadIdx.x; i < H4; i += blockDim.x) { const float4 v = y[base + i]; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)(4 * H4) + eps);
  if (NV > 0) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < H4) {
        float4 h = hidden[base + i];
        const float4 g = w[i];
        h.x += keep[j].x * inv * g.x; h.y += keep[j].y * inv * g.y; h.z += keep[j].z * inv * g.z; h.w += keep[j].w * inv * g.w;
        hidden[base + i] = h;
      }
    }
  } else {
    for (int i = threadIdx.x; i < H4; i += blockDim.x) {
      float4 h = hidden[base + i];
      const float4 v = y[base + i], g = w[i];
      h.x += v.x * inv * g.x; h.y += v.y * inv * g.y; h.z += v.z * inv * g.z; h.w += v.w * inv * g.w;
      hidden[base + i] = h;
    }
  }
}

extern "C" int odi_rmsnorm_add(float* hidden, const float* y, const float* w, int n, int H, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H % 4 == 0 && ((uintptr_t)hidden | (uintptr_t)y | (uintptr_t)w) % 16 == 0) {
    const int H4 = H / 4;
    const int vthreads = H4 >= 1024 ? 512 : (H4 >= 256 ? 256 : (H4 >= 128 ? 128 : 64));
    const int per = (H4 + vthreads - 1) / vthreads;
    if (per <= 1) odi_rc = launch_pdl((rmsnorm_add_vec_kernel<1>), dim3(n), dim3(vthreads), 0, stream, (float4*)hidden, (const float4*)y, (const float4*)w, H4, eps);
    else if (per <= 2) odi_rc = launch_pdl((rmsnorm_add_vec_kernel<2>), dim3(n), dim3(vthreads), 0, stream, (float4*)hidden, (const float4*)y, (const float4*)w, H4, eps);
    else if (per <= 4) odi_rc = launch_pdl((rmsnorm_add_vec_kernel<4>), dim3(n), dim3(vthreads), 0, stream, (float4*)hidden, (const float4*)y, (const float4*)w, H4, eps);
    else odi_rc = launch_pdl((rmsnorm_add_vec_kernel<0>), dim3(n), dim3(vthreads), 0, stream, (float4*)hidden, (const float4*)y, (const float4*)w, H4, eps);
    return launch_status();
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  odi_rc = launch_pdl((rmsnorm_add_kernel), dim3(n), dim3(threads), 0, stream, hidden, y, w, H, eps);
  return launch_status();
}

// rmsnorm_add and the norm that the next sublayer takes of the sum, in one pass: the row of the sum stays in
// registers (NV float4 per thread).  h += y * rsqrt(mean(y^2) + eps) * w; out = T(h * rsqrt(mean(h^2) + eps2) * w2).
template <typename T, int NV>
__global__ void rmsnorm_add_norm_kernel(float4* __restrict__ hidden, const float4* __restrict__ y, const float4* __restrict__ w,
                                        float eps, const float4* __restrict__ w2, float eps2, T* __restrict__ out, int H4) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * H4;
  float4 keep[NV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    keep[j] = i < H4 ? y[base + i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)(4 * H4) + eps);
  float ss2 = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < H4) {
      float4 h = hidden[base + i];
      const float4 g = w[i];
      h.x += keep[j].x * inv * g.x; h.y += keep[j].y * inv * g.y; h.z += keep[j].z * inv * g.z; h.w += keep[j].w * inv * g.w;
      hidden[base + i] = h;
      keep[j] = h;
      ss2 += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
    }
  }
  ss2 = block_sum(ss2, scratch);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)(4 * H4) + eps2);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < H4) {
      const float4 g = w2[i];
      const float4 v = make_float4(keep[j].x * inv2 * g.x, keep[j].y * inv2 * g.y, keep[j].z * inv2 * g.z, keep[j].w * inv2 * g.w);
      if (sizeof(T) == 4) {
        ((float4*)out)[base + i] = v;
      } else {
        uint2 packed;
        *(__nv_bfloat162*)&packed.x = __floats2bfloat162_rn(v.x, v.y);
        *(__nv_bfloat162*)&packed.y = __floats2bfloat162_rn(v.z, v.w);
        ((uint2*)out)[base + i] = packed;
      }
    }
  }
}

extern "C" int odi_rmsnorm_add_norm(float* hidden, const float* y, const float* w, float eps, const float* w2, float eps2,
                                    void* out, int n, int H, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H % 4 != 0 || H > 8192 || ((uintptr_t)hidden | (uintptr_t)y | (uintptr_t)w | (uintptr_t)w2 | (uintptr_t)out) % 16 != 0)
    return ODI_ERR_UNSUPPORTED;
  const int H4 = H / 4;
  const int threads = H4 >= 1024 ? 512 : (H4 >= 256 ? 256 : (H4 >= 128 ? 128 : 64));
  const int per = (H4 + threads - 1) / threads;
#define ODI_RAN(T, NV) odi_rc = launch_pdl((rmsnorm_add_norm_kernel<T, NV>), dim3(n), dim3(threads), 0, stream, (float4*)hidden, \
    (const float4*)y, (const float4*)w, eps, (const float4*)w2, eps2, (T*)out, H4)
  if (dtype == 0) { if (per <= 1) ODI_RAN(float, 1); else if (per <= 2) ODI_RAN(float, 2); else ODI_RAN(float, 4); }
  else { if (per <= 1) ODI_RAN(bf16, 1); else if (per <= 2) ODI_RAN(bf16, 2); else ODI_RAN(bf16, 4); }
#undef ODI_RAN
  return launch_status();
}

// acc[t] += sigmoid(x[t] . g) * y[t]; the dot product in fp32 over the row of x (T), y fp32 or T.
template <typename T, typename Y>
__global__ void gated_row_add_kernel(float* __restrict__ acc, const Y* __restrict__ y, const T* __restrict__ x,
                                     const T* __restrict__ g, int H, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  float dot = 0.f;
  for (int i = threadIdx.x; i < K; i += blockDim.x) dot = fmaf(to_f<T>(x[t * K + i]), to_f<T>(g[i]), dot);
  dot = block_sum(dot, scratch);
  const float gate = 1.0f / (1.0f + expf(-dot));
  for (int i = threadIdx.x; i < H; i += blockDim.x) acc[t * H + i] = fmaf(gate, to_f<Y>(y[t * H + i]), acc[t * H + i]);
}

// bf16 x and gate with fp32 or bf16 y, eight lanes at a time (K and H multiples of 8, aligned rows).
template <typename Y>
__global__ void gated_row_add_vec_kernel(float* __restrict__ acc, const Y* __restrict__ y, const bf16* __restrict__ x,
                                         const bf16* __restrict__ g, int H, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  float dot = 0.f;
  for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) {
    const uint4 xr = *(const uint4*)(x + t * K + i), gr = *(const uint4*)(g + i);
    const __nv_bfloat162* xh = (const __nv_bfloat162*)&xr;
    const __nv_bfloat162* gh = (const __nv_bfloat162*)&gr;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(xh[e]), b = __bfloat1622float2(gh[e]);
      dot = fmaf(a.x, b.x, dot); dot = fmaf(a.y, b.y, dot);
    }
  }
  dot = block_sum(dot, scratch);
  const float gate = 1.0f / (1.0f + expf(-dot));
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8];
    if (sizeof(Y) == 4) {
      const float4 lo = *(const float4*)((const float*)y + t * H + i), hi = *(const float4*)((const float*)y + t * H + i + 4);
      v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    } else {
      const uint4 raw = *(const uint4*)((const bf16*)y + t * H + i);
      const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw;
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h2[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
    }
    float4* dst = (float4*)(acc + t * H + i);
    float4 lo = dst[0], hi = dst[1];
    lo.x = fmaf(gate, v[0], lo.x); lo.y = fmaf(gate, v[1], lo.y); lo.z = fmaf(gate, v[2], lo.z); lo.w = fmaf(gate, v[3], lo.w);
    hi.x = fmaf(gate, v[4], hi.x); hi.y = fmaf(gate, v[5], hi.y); hi.z = fmaf(gate, v[6], hi.z); hi.w = fmaf(gate, v[7], hi.w);
    dst[0] = lo; dst[1] = hi;
  }
}

// y_is_t: y has the dtype of x; else it is fp32.
extern "C" int odi_gated_row_add(float* acc, const void* y, const void* x, const void* g, int n, int H, int K, int y_is_t,
                                 int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (dtype == 1 && H % 8 == 0 && K % 8 == 0 && ((uintptr_t)acc | (uintptr_t)y | (uintptr_t)x | (uintptr_t)g) % 16 == 0) {
    const int vthreads = H >= 2048 ? 256 : 128;
    if (y_is_t) odi_rc = launch_pdl((gated_row_add_vec_kernel<bf16>), dim3(n), dim3(vthreads), 0, stream, acc, (const bf16*)y, (const bf16*)x, (const bf16*)g, H, K);
    else odi_rc = launch_pdl((gated_row_add_vec_kernel<float>), dim3(n), dim3(vthreads), 0, stream, acc, (const float*)y, (const bf16*)x, (const bf16*)g, H, K);
    return launch_status();
  }
  if (dtype == 0) odi_rc = launch_pdl((gated_row_add_kernel<float, float>), dim3(n), dim3(threads), 0, stream, acc, (const float*)y, (const float*)x, (const float*)g, H, K);
  else if (y_is_t) odi_rc = launch_pdl((gated_row_add_kernel<bf16, bf16>), dim3(n), dim3(threads), 0, stream, acc, (const bf16*)y, (const bf16*)x, (const bf16*)g, H, K);
  else odi_rc = launch_pdl((gated_row_add_kernel<bf16, float>), dim3(n), dim3(threads), 0, stream, acc, (const float*)y, (const bf16*)x, (const bf16*)g, H, K);
  return launch_status();
}
