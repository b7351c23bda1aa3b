// Head preparation of latent attention: what lies between the fused query / down projection and the
// attention kernel over the compressed cache.
//
// One block per token reads its row of the projection output
//   [ head 0: d plain lanes, r rotated lanes | head 1 ... | R latent lanes | r shared rotated key lanes ]
// (cache rows and absorbed queries may be wider than R + r, `row` lanes, so that R + r need not be a multiple of
// four; the lanes beyond are zero on both sides and add nothing to a score)
// and
//  * norms the R latent lanes (RMS over R in fp32, times a plain weight, eps inside the root), rounds them
//    once to T and writes them to lanes 0..R-1 of the token's row in the paged cache;
//  * rotates the shared key lanes and writes them to lanes R..R+r-1 of that row;
//  * rotates each head's r query lanes and writes them to lanes R..R+r-1 of that head's row of the
//    absorbed query [tokens, heads, R + r] (lanes 0..R-1 are left to the product that folds the key
//    up-projection into the query).
// Rotation: lanes (2i, 2i+1), i < rot_dims / 2, turn by the angle whose cosine and sine the step's
// tables hold (fp32); lanes from rot_dims on pass unchanged.  `interleaved == 0` pairs lane i with lane
// i + rot_dims / 2 instead.
#include "common.cuh"

struct LatentPrepArgs {
  const void* proj;      // [n_tokens, ld] in T
  void* q_abs;           // [n_tokens, heads, R + r] in T
  void* pool;            // [pages, 1, page_size, R + r] in T
  const float* norm_w;   // [R]
  const float* cos_t;    // [n_tokens, rot_dims / 2]
  const float* sin_t;
  const int* tok_seq;
  const int* tok_pos;
  const int* page_start;
  const int* page_ids;
  int n_tokens, ld, heads, d, r, R, rot_dims, interleaved, page_size, ring_pages, write_cache;
  float eps;
  void* latent_out;      // null, or [n_tokens, R] in T: the normed latent once more, rows side by side
  void* key_rot_out;     // null, or [n_tokens, r] in T: the rotated shared key lanes once more
  int row;               // lanes of a cache row and of a head's absorbed query: R + r, or more (lanes beyond stay zero)
  const void* down;      // null: the R + r lanes of the down projection follow the heads in `proj`; else
  int ld_down;           // [n_tokens, ld_down] in T, the lanes at its start (queries that come from a product of their own)
  int has_down;          // 0: a layer that reads another layer's cache rows: only the queries are prepared
};

__device__ __forceinline__ void rotated_pair(int lane, int rot_dims, int interleaved, int* a, int* b, int* i) {
  // the pair that `lane` belongs to: (*a, *b) with angle index *i
  if (interleaved) { *i = lane >> 1; *a = 2 * *i; *b = *a + 1; }
  else { const int half = rot_dims >> 1; *i = lane < half ? lane : lane - half; *a = *i; *b = *i + half; }
}

template <typename T>
__device__ __forceinline__ float rotate_lane(const T* src, int lane, const LatentPrepArgs& a, const float* cs,
                                             const float* sn) {
  if (lane >= a.rot_dims) return to_f<T>(src[lane]);
  int pa, pb, i;
  rotated_pair(lane, a.rot_dims, a.interleaved, &pa, &pb, &i);
  const float u = to_f<T>(src[pa]), v = to_f<T>(src[pb]);
  return lane == pa ? u * cs[i] - v * sn[i] : v * cs[i] + u * sn[i];
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(LatentPrepArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const T* row = (const T*)a.proj + (size_t)t * a.ld;
  const int q_width = a.heads * (a.d + a.r);
  const T* down = a.down != nullptr ? (const T*)a.down + (size_t)t * a.ld_down : row + q_width;
  const float* cs = a.cos_t + (size_t)t * (a.rot_dims / 2);
  const float* sn = a.sin_t + (size_t)t * (a.rot_dims / 2);
  const int W = a.row;

  float inv = 0.f;
  if (a.has_down) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) { const float v = to_f<T>(down[i]); ss += v * v; }
    ss = block_sum(ss, scratch);
    inv = 1.0f / sqrtf(ss / (float)a.R + a.eps);
  }

  if (a.has_down && a.write_cache) {
    const int seq = a.tok_seq[t], pos = a.tok_pos[t];
    const int page = a.page_ids[a.page_start[seq] + page_slot_of(pos, a.page_size, a.ring_pages)];
    T* dst = (T*)a.pool + ((size_t)page * a.page_size + (pos % a.page_size)) * W;
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) dst[i] = from_f<T>(to_f<T>(down[i]) * inv * a.norm_w[i]);
    for (int i = threadIdx.x; i < a.r; i += blockDim.x) dst[a.R + i] = from_f<T>(rotate_lane<T>(down + a.R, i, a, cs, sn));
  }
  if (a.has_down && a.latent_out != nullptr) {
    T* lat = (T*)a.latent_out + (size_t)t * a.R;
    T* kr = (T*)a.key_rot_out + (size_t)t * a.r;
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) lat[i] = from_f<T>(to_f<T>(down[i]) * inv * a.norm_w[i]);
    for (int i = threadIdx.x; i < a.r; i += blockDim.x) kr[i] = from_f<T>(rotate_lane<T>(down + a.R, i, a, cs, sn));
  }
  T* q_out = (T*)a.q_abs + (size_t)t * a.heads * W;
  for (int i = threadIdx.x; i < a.heads * a.r; i += blockDim.x) {
    const int h = i / a.r, lane = i % a.r;
    q_out[(size_t)h * W + a.R + lane] = from_f<T>(rotate_lane<T>(row + h * (a.d + a.r) + a.d, lane, a, cs, sn));
  }
}

// Whole heads for a prompt that starts its sequence: the attention kernels for ordinary heads then serve it.
// Per (token, head): query [plain lanes | rotated lanes | zeros] into q_full [tokens, heads, Dh]; key
// [up-projected plain lanes | the shared rotated lanes | zeros] and value [up-projected lanes | zeros] into
// pools [pages, heads, page_size, Dh] of the step's own, where sequence s holds pages page_start[s].. in order.
struct LatentExpandArgs {
  const void* proj;      // [n_tokens, ld]: per head d plain query lanes (then r lanes that are not read here)
  const void* q_abs;     // [n_tokens, heads, row]: the rotated query lanes at R..
  const void* k_plain;   // [n_tokens, heads * d]
  const void* key_rot;   // [n_tokens, r]
  const void* v;         // [n_tokens, heads * dv]
  void* q_full;
  void* k_pool;
  void* v_pool;
  const int* tok_seq;
  const int* cu_q;
  const int* page_start;
  int n_tokens, ld, heads, d, r, R, dv, Dh, page_size, row;
};

template <typename T>
__global__ void __launch_bounds__(128)
latent_expand_kernel(LatentExpandArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int seq = a.tok_seq[t];
  const int li = t - a.cu_q[seq];
  const size_t slot = ((size_t)(a.page_start[seq] + li / a.page_size) * a.heads + h) * a.page_size + li % a.page_size;
  const T* qp = (const T*)a.proj + (size_t)t * a.ld + h * (a.d + a.r);
  const T* qr = (const T*)a.q_abs + ((size_t)t * a.heads + h) * a.row + a.R;
  const T* kp = (const T*)a.k_plain + ((size_t)t * a.heads + h) * a.d;
  const T* kr = (const T*)a.key_rot + (size_t)t * a.r;
  const T* vp = (const T*)a.v + ((size_t)t * a.heads + h) * a.dv;
  T* q = (T*)a.q_full + ((size_t)t * a.heads + h) * a.Dh;
  T* k = (T*)a.k_pool + slot * a.Dh;
  T* v = (T*)a.v_pool + slot * a.Dh;
  const T zero = from_f<T>(0.f);
  for (int i = threadIdx.x; i < a.Dh; i += blockDim.x) {
    q[i] = i < a.d ? qp[i] : (i < a.d + a.r ? qr[i - a.d] : zero);
    k[i] = i < a.d ? kp[i] : (i < a.d + a.r ? kr[i - a.d] : zero);
    v[i] = i < a.dv ? vp[i] : zero;
  }
}

// The same in 16-byte pieces, a block per token: every size a multiple of a piece's lanes, every pointer aligned.
template <typename T>
__global__ void __launch_bounds__(256)
latent_expand_vec_kernel(LatentExpandArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CH = 16 / (int)sizeof(T);      // lanes of a piece
  const int t = blockIdx.x;
  const int seq = a.tok_seq[t];
  const int li = t - a.cu_q[seq];
  const size_t page = (size_t)(a.page_start[seq] + li / a.page_size) * a.heads;
  const int in_page = li % a.page_size;
  const int pieces = a.Dh / CH;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const T* kr = (const T*)a.key_rot + (size_t)t * a.r;
  for (int i = threadIdx.x; i < a.heads * pieces; i += blockDim.x) {
    const int h = i / pieces, lane = (i % pieces) * CH;
    const size_t slot = (page + h) * a.page_size + in_page;
    const T* qp = (const T*)a.proj + (size_t)t * a.ld + h * (a.d + a.r);
    const T* qr = (const T*)a.q_abs + ((size_t)t * a.heads + h) * a.row + a.R;
    const T* kp = (const T*)a.k_plain + ((size_t)t * a.heads + h) * a.d;
    const T* vp = (const T*)a.v + ((size_t)t * a.heads + h) * a.dv;
    const bool plain = lane < a.d, rotated = !plain && lane < a.d + a.r;
    const uint4 q = plain ? *(const uint4*)(qp + lane) : (rotated ? *(const uint4*)(qr + lane - a.d) : zero);
    const uint4 k = plain ? *(const uint4*)(kp + lane) : (rotated ? *(const uint4*)(kr + lane - a.d) : zero);
    const uint4 v = lane < a.dv ? *(const uint4*)(vp + lane) : zero;
    *(uint4*)((T*)a.q_full + ((size_t)t * a.heads + h) * a.Dh + lane) = q;
    *(uint4*)((T*)a.k_pool + slot * a.Dh + lane) = k;
    *(uint4*)((T*)a.v_pool + slot * a.Dh + lane) = v;
  }
}

extern "C" int odi_latent_expand(const LatentExpandArgs* args, int dtype, cudaStream_t stream) {
  const LatentExpandArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (a.Dh < a.d + a.r || a.Dh < a.dv || a.heads <= 0 || a.heads > 65535) return ODI_ERR_ARGUMENT;
  const int ch = dtype == 0 ? 4 : 8;
  const uintptr_t pointers = (uintptr_t)a.proj | (uintptr_t)a.q_abs | (uintptr_t)a.k_plain | (uintptr_t)a.key_rot |
                             (uintptr_t)a.v | (uintptr_t)a.q_full | (uintptr_t)a.k_pool | (uintptr_t)a.v_pool;
  if ((a.d | a.r | a.dv | a.Dh | a.ld | a.row | a.R) % ch == 0 && (pointers & 15) == 0) {
    if (dtype == 0) odi_rc = launch_pdl((latent_expand_vec_kernel<float>), dim3(a.n_tokens), dim3(256), 0, stream, a);
    else odi_rc = launch_pdl((latent_expand_vec_kernel<bf16>), dim3(a.n_tokens), dim3(256), 0, stream, a);
    return launch_status();
  }
  const dim3 grid(a.n_tokens, a.heads);
  if (dtype == 0) odi_rc = launch_pdl((latent_expand_kernel<float>), grid, dim3(128), 0, stream, a);
  else odi_rc = launch_pdl((latent_expand_kernel<bf16>), grid, dim3(128), 0, stream, a);
  return launch_status();
}

extern "C" int odi_latent_prep(const LatentPrepArgs* args, int dtype, cudaStream_t stream) {
  const LatentPrepArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (a.rot_dims % 2 != 0 || a.rot_dims > a.r || a.R <= 0 || a.heads <= 0 || a.row < a.R + a.r) return ODI_ERR_ARGUMENT;
  if (!a.has_down && (a.write_cache || a.latent_out != nullptr)) return ODI_ERR_ARGUMENT;
  if (dtype == 0) odi_rc = launch_pdl((latent_prep_kernel<float>), dim3(a.n_tokens), dim3(128), 0, stream, a);
  else odi_rc = launch_pdl((latent_prep_kernel<bf16>), dim3(a.n_tokens), dim3(128), 0, stream, a);
  return launch_status();
}


// ---------------------------------------------------------------------------------
// A latent in front of a projection: out[t, :] = T(in[t, col .. col + Q) / sqrt(mean of squares + eps) * w),
// the statistics and the scaling in fp32, one rounding.  `in` rows are ld lanes apart (the latent is a slice of a
// wider product).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
slice_norm_kernel(const T* __restrict__ in, const float* __restrict__ w, T* __restrict__ out, int ld, int col, int Q,
                  float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const T* src = in + (size_t)blockIdx.x * ld + col;
  float ss = 0.f;
  for (int i = threadIdx.x; i < Q; i += blockDim.x) { const float v = to_f<T>(src[i]); ss += v * v; }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)Q + eps);
  T* dst = out + (size_t)blockIdx.x * Q;
  for (int i = threadIdx.x; i < Q; i += blockDim.x) dst[i] = from_f<T>(to_f<T>(src[i]) * inv * w[i]);
}

extern "C" int odi_slice_norm(const void* in, const float* w, void* out, int rows, int ld, int col, int Q, float eps,
                              int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (Q <= 0 || col < 0 || col + Q > ld) return ODI_ERR_ARGUMENT;
  if (dtype == 0) odi_rc = launch_pdl((slice_norm_kernel<float>), dim3(rows), dim3(128), 0, stream, (const float*)in, w, (float*)out, ld, col, Q, eps);
  else odi_rc = launch_pdl((slice_norm_kernel<bf16>), dim3(rows), dim3(128), 0, stream, (const bf16*)in, w, (bf16*)out, ld, col, Q, eps);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// An output gate on the heads: x[t, h, i] *= sigmoid(gate[t, col + h dv + i]) for i < dv; a head of x has `lanes`
// lanes (>= dv; the ones beyond are left as they are), rows of `gate` are ld lanes apart.  The sigmoid and the
// product in fp32, one rounding.
// ---------------------------------------------------------------------------------
// per_head: the gate has one lane per head (at col + h) that multiplies all of the head's lanes.
template <typename T>
__global__ void gate_heads_kernel(T* __restrict__ x, const T* __restrict__ gate, long total, int heads, int dv, int lanes,
                                  int ld, int col, int per_head) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int i = (int)(idx % dv);
  const int h = (int)((idx / dv) % heads);
  const long t = idx / ((long)dv * heads);
  const float gv = to_f<T>(gate[t * ld + col + (per_head ? h : h * dv + i)]);
  T* p = x + (t * heads + h) * lanes + i;
  *p = from_f<T>(to_f<T>(*p) / (1.0f + expf(-gv)));
}

// Eight bf16 lanes a thread (dv, lanes, ld and col multiples of 8, aligned tensors).
__global__ void gate_heads_vec_kernel(bf16* __restrict__ x, const bf16* __restrict__ gate, long total8, int heads, int dv,
                                      int lanes, int ld, int col) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per = dv >> 3;
  const int i = (int)(idx % per) * 8;
  const int h = (int)((idx / per) % heads);
  const long t = idx / ((long)per * heads);
  const uint4 graw = *(const uint4*)(gate + t * ld + col + h * dv + i);
  bf16* p = x + (t * heads + h) * lanes + i;
  uint4 xraw = *(const uint4*)p;
  const __nv_bfloat162* g2 = (const __nv_bfloat162*)&graw;
  __nv_bfloat162* x2 = (__nv_bfloat162*)&xraw;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 g = __bfloat1622float2(g2[e]), v = __bfloat1622float2(x2[e]);
    x2[e] = __floats2bfloat162_rn(v.x / (1.0f + expf(-g.x)), v.y / (1.0f + expf(-g.y)));
  }
  *(uint4*)p = xraw;
}

extern "C" int odi_gate_heads(void* x, const void* gate, int rows, int heads, int dv, int lanes, int ld, int col,
                              int per_head, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || dv <= 0 || lanes < dv || col < 0 || col + heads * (per_head ? 1 : dv) > ld) return ODI_ERR_ARGUMENT;
  const long total = (long)rows * heads * dv;
  if (!per_head && dtype == 1 && dv % 8 == 0 && lanes % 8 == 0 && ld % 8 == 0 && col % 8 == 0 && (((uintptr_t)x | (uintptr_t)gate) & 15) == 0) {
    const long total8 = total / 8, vblocks = (total8 + 255) / 256;
    if (vblocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
    odi_rc = launch_pdl((gate_heads_vec_kernel), dim3((unsigned)vblocks), dim3(256), 0, stream, (bf16*)x, (const bf16*)gate, total8, heads, dv, lanes, ld, col);
    return launch_status();
  }
  const long blocks = (total + 255) / 256;
  if (blocks > 2147483647L) return ODI_ERR_UNSUPPORTED;
  if (dtype == 0) odi_rc = launch_pdl((gate_heads_kernel<float>), dim3((unsigned)blocks), dim3(256), 0, stream, (float*)x, (const float*)gate, total, heads, dv, lanes, ld, col, per_head);
  else odi_rc = launch_pdl((gate_heads_kernel<bf16>), dim3((unsigned)blocks), dim3(256), 0, stream, (bf16*)x, (const bf16*)gate, total, heads, dv, lanes, ld, col, per_head);
  return launch_status();
}
