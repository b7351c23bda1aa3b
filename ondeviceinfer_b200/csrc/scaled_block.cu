// Kernels of a block whose mixer and feed-forward read two norms of the same stream side by side and whose
// outputs are scaled lane by lane before they are added,
//   x <- x + s1 * mixer(norm1(x)) + s2 * ff(norm2(x)),
// of a per-layer input that is looked up by token id, and of two mixers that run side by side:
//
//  * dual_norm: out1 = cast(x * r * w1), out2 = cast(x * r * w2), r = 1 / sqrt(mean(x^2) + eps): both norms of a row
//    from one sum of squares and one read of the stream (the weights hold what multiplies a lane, an offset of one
//    included); fp32 arithmetic, one rounding each.
//  * scaled_add2: x += a * s1 (+ b * s2), fp32, s1 and s2 one number per lane; optionally the new row once more in T.
//  * weighted_sum: out = ca * a + cb * b on fp32 rows (two mixers' outputs and a factor each).
//  * gated_lookup: out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col + j] in T (fp32 arithmetic, one rounding):
//    a gate on the stream times a row that the token id picks.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
dual_norm_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ w2, T* __restrict__ out1,
                 T* __restrict__ out2, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  const float* row = x + t * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = row[i] * inv;
    out1[t * H + i] = from_f<T>(v * w1[i]);
    out2[t * H + i] = from_f<T>(v * w2[i]);
  }
}

// H a multiple of 4 and at most 4 * 256 * NV: the row stays in registers between the two passes.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
dual_norm_vec_kernel(const float4* __restrict__ x, const float4* __restrict__ w1, const float4* __restrict__ w2,
                     T* __restrict__ out1, T* __restrict__ out2, int H4, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < NV; ++r) {
    const int i = threadIdx.x + r * 256;
    if (i < H4) {
      v[r] = x[t * H4 + i];
      ss += v[r].x * v[r].x + v[r].y * v[r].y + v[r].z * v[r].z + v[r].w * v[r].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)(4 * H4) + eps);
#pragma unroll
  for (int r = 0; r < NV; ++r) {
    const int i = threadIdx.x + r * 256;
    if (i < H4) {
      const float4 a = w1[i], b = w2[i];
      const float4 n = make_float4(v[r].x * inv, v[r].y * inv, v[r].z * inv, v[r].w * inv);
      T* o1 = out1 + (t * H4 + i) * 4;
      T* o2 = out2 + (t * H4 + i) * 4;
      o1[0] = from_f<T>(n.x * a.x); o1[1] = from_f<T>(n.y * a.y); o1[2] = from_f<T>(n.z * a.z); o1[3] = from_f<T>(n.w * a.w);
      o2[0] = from_f<T>(n.x * b.x); o2[1] = from_f<T>(n.y * b.y); o2[2] = from_f<T>(n.z * b.z); o2[3] = from_f<T>(n.w * b.w);
    }
  }
}

extern "C" int odi_dual_norm(const float* x, const float* w1, const float* w2, void* out1, void* out2, int n, int H, float eps,
                             int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0) return ODI_ERR_ARGUMENT;
  const bool vec = H % 4 == 0 && H <= 4 * 256 * 8 && (((uintptr_t)x | (uintptr_t)w1 | (uintptr_t)w2) & 15) == 0;
  if (vec) {
    const int H4 = H / 4, nv = (H4 + 255) / 256;
#define ODI_DN(T, NV) odi_rc = launch_pdl((dual_norm_vec_kernel<T, NV>), dim3(n), dim3(256), 0, stream, (const float4*)x, \
                                          (const float4*)w1, (const float4*)w2, (T*)out1, (T*)out2, H4, eps)
    if (dtype == 0) { if (nv <= 1) ODI_DN(float, 1); else if (nv <= 2) ODI_DN(float, 2); else if (nv <= 4) ODI_DN(float, 4); else ODI_DN(float, 8); }
    else { if (nv <= 1) ODI_DN(bf16, 1); else if (nv <= 2) ODI_DN(bf16, 2); else if (nv <= 4) ODI_DN(bf16, 4); else ODI_DN(bf16, 8); }
#undef ODI_DN
    return launch_status();
  }
  if (dtype == 0) odi_rc = launch_pdl((dual_norm_kernel<float>), dim3(n), dim3(256), 0, stream, x, w1, w2, (float*)out1, (float*)out2, H, eps);
  else odi_rc = launch_pdl((dual_norm_kernel<bf16>), dim3(n), dim3(256), 0, stream, x, w1, w2, (bf16*)out1, (bf16*)out2, H, eps);
  return launch_status();
}

template <typename T>
__global__ void __launch_bounds__(256)
scaled_add2_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ s1, const float* __restrict__ b,
                   const float* __restrict__ s2, T* __restrict__ copy, long n, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int lane = (int)(i % H);
  float v = fmaf(a[i], s1[lane], x[i]);
  if (b != nullptr) v = fmaf(b[i], s2[lane], v);
  x[i] = v;
  if (copy != nullptr) copy[i] = from_f<T>(v);
}

// Four lanes a thread (H a multiple of 4, aligned tensors): the same arithmetic.
template <typename T>
__global__ void __launch_bounds__(256)
scaled_add2_vec_kernel(float4* __restrict__ x, const float4* __restrict__ a, const float4* __restrict__ s1, const float4* __restrict__ b,
                       const float4* __restrict__ s2, T* __restrict__ copy, long n4, int H4) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const int lane = (int)(i % H4);
  float4 v = x[i];
  const float4 av = a[i], sv = s1[lane];
  v.x = fmaf(av.x, sv.x, v.x); v.y = fmaf(av.y, sv.y, v.y); v.z = fmaf(av.z, sv.z, v.z); v.w = fmaf(av.w, sv.w, v.w);
  if (b != nullptr) {
    const float4 bv = b[i], tv = s2[lane];
    v.x = fmaf(bv.x, tv.x, v.x); v.y = fmaf(bv.y, tv.y, v.y); v.z = fmaf(bv.z, tv.z, v.z); v.w = fmaf(bv.w, tv.w, v.w);
  }
  x[i] = v;
  if (copy != nullptr) {
    T* c = copy + i * 4;
    c[0] = from_f<T>(v.x); c[1] = from_f<T>(v.y); c[2] = from_f<T>(v.z); c[3] = from_f<T>(v.w);
  }
}

extern "C" int odi_scaled_add2(float* x, const float* a, const float* s1, const float* b, const float* s2, void* copy, long rows,
                               int H, int dtype, cudaStream_t stream) {
  const long n = rows * H;
  if (n <= 0) return 0;
  if (b != nullptr && s2 == nullptr) return ODI_ERR_ARGUMENT;
  if (H % 4 == 0 && (((uintptr_t)x | (uintptr_t)a | (uintptr_t)s1 | (uintptr_t)b | (uintptr_t)s2 | (uintptr_t)copy) & 15) == 0) {
    const long n4 = n / 4, vblocks = (n4 + 255) / 256;
    if (vblocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
    if (dtype == 0) odi_rc = launch_pdl((scaled_add2_vec_kernel<float>), dim3((unsigned)vblocks), dim3(256), 0, stream, (float4*)x, (const float4*)a, (const float4*)s1, (const float4*)b, (const float4*)s2, (float*)copy, n4, H / 4);
    else odi_rc = launch_pdl((scaled_add2_vec_kernel<bf16>), dim3((unsigned)vblocks), dim3(256), 0, stream, (float4*)x, (const float4*)a, (const float4*)s1, (const float4*)b, (const float4*)s2, (bf16*)copy, n4, H / 4);
    return launch_status();
  }
  const long blocks = (n + 255) / 256;
  if (blocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
  if (dtype == 0) odi_rc = launch_pdl((scaled_add2_kernel<float>), dim3((unsigned)blocks), dim3(256), 0, stream, x, a, s1, b, s2, (float*)copy, n, H);
  else odi_rc = launch_pdl((scaled_add2_kernel<bf16>), dim3((unsigned)blocks), dim3(256), 0, stream, x, a, s1, b, s2, (bf16*)copy, n, H);
  return launch_status();
}

__global__ void __launch_bounds__(256)
weighted_sum_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, long n, float ca, float cb) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = fmaf(cb, b[i], ca * a[i]);
}

__global__ void __launch_bounds__(256)
weighted_sum_vec_kernel(float4* __restrict__ out, const float4* __restrict__ a, const float4* __restrict__ b, long n4, float ca, float cb) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 av = a[i], bv = b[i];
  out[i] = make_float4(fmaf(cb, bv.x, ca * av.x), fmaf(cb, bv.y, ca * av.y), fmaf(cb, bv.z, ca * av.z), fmaf(cb, bv.w, ca * av.w));
}

extern "C" int odi_weighted_sum(float* out, const float* a, const float* b, long n, float ca, float cb, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 == 0 && (((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) & 15) == 0) {
    const long vblocks = (n / 4 + 255) / 256;
    if (vblocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
    odi_rc = launch_pdl(weighted_sum_vec_kernel, dim3((unsigned)vblocks), dim3(256), 0, stream, (float4*)out, (const float4*)a, (const float4*)b, n / 4, ca, cb);
    return launch_status();
  }
  const long blocks = (n + 255) / 256;
  if (blocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
  odi_rc = launch_pdl(weighted_sum_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, out, a, b, n, ca, cb);
  return launch_status();
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_lookup_kernel(const T* __restrict__ z, const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out, long n,
                    int dim, int ld_table, int col) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long t = i / dim;
  const int j = (int)(i % dim);
  const float v = to_f<T>(z[i]);
  const float g = 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));
  out[i] = from_f<T>(g * to_f<T>(table[(size_t)ids[t] * ld_table + col + j]));
}

extern "C" int odi_gated_lookup(const void* z, const void* table, const int* ids, void* out, long rows, int dim, int ld_table,
                                int col, int dtype, cudaStream_t stream) {
  const long n = rows * dim;
  if (n <= 0) return 0;
  if (col < 0 || col + dim > ld_table) return ODI_ERR_ARGUMENT;
  const long blocks = (n + 255) / 256;
  if (blocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
  if (dtype == 0) odi_rc = launch_pdl((gated_lookup_kernel<float>), dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)z, (const float*)table, ids, (float*)out, n, dim, ld_table, col);
  else odi_rc = launch_pdl((gated_lookup_kernel<bf16>), dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)z, (const bf16*)table, ids, (bf16*)out, n, dim, ld_table, col);
  return launch_status();
}

// out = cast(x) for fp32 rows (the stream once more in the compute dtype, for a product that reads it).
template <typename T>
__global__ void __launch_bounds__(256)
cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long n) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f<T>(x[i]);
}

extern "C" int odi_cast_rows(const float* x, void* out, long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long blocks = (n + 255) / 256;
  if (blocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
  if (dtype == 0) odi_rc = launch_pdl((cast_rows_kernel<float>), dim3((unsigned)blocks), dim3(256), 0, stream, x, (float*)out, n);
  else odi_rc = launch_pdl((cast_rows_kernel<bf16>), dim3((unsigned)blocks), dim3(256), 0, stream, x, (bf16*)out, n);
  return launch_status();
}
