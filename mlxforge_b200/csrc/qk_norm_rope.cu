// Queries, keys and values on their way from the projection into the attention, for mixers that
// normalise queries and keys over the WHOLE projection (all heads at once) before the rotation:
//
//   q = rms(Wq h + bq) gq ,  k = rms(Wk h + bk) gk         (one root mean square over all rows of q, one over k)
//   rotation of the first `rot` channels of every head, pair (i, i + rot/2), by position * inv[i];
//   cosine and sine both times `magnitude`
//   values: the row's own value heads, optionally rotated over all their vd channels (pair (m, m + vd/2)
//   by position * vinv[m]), or the keys as projected (with their bias, before norm and rotation)
//
// One block per token.  A row of `proj` (rows `ld` elements apart) holds the query heads, the key
// heads and (own values) the value heads.  Biases, sums of squares, norms and rotations are 32-bit
// (angles in double where a float64 table is given); queries go to q_out [T, n_heads * hd], keys and
// values into their pages (value pages are vd wide).
//
// rotate_rows turns the heads of finished rows by sign * position (an attention output over rotated
// values is turned back by its query's position).
#include "rotary.cuh"

struct QkPrepare {
  int n_heads, n_kv, hd, vd, rot;
  int v_mode;                 // 0: own values, 1: the keys as projected
  float eps, magnitude;
  const float* bias;          // [nq + nk (+ nv)] or null
  const float* q_w;           // [nq] or null (no norm)
  const float* k_w;           // [nk] or null
  const float* inv_f;         // [rot/2]
  const double* inv_d;
  const float* vinv_f;        // [vd/2] or null: values are not rotated
  const double* vinv_d;
};

template <typename TP, typename T>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const TP* __restrict__ proj, int ld, QkPrepare p, const int* __restrict__ positions,
                    const int* __restrict__ seq_of_token, PagedView pk, PagedView pvv, T* __restrict__ q_out,
                    T* __restrict__ k_pool, T* __restrict__ v_pool, int write_kv) {
  extern __shared__ float qs[];     // row [nq + nk + nv], then cos/sin of the keys' and of the values' rotation
  __shared__ float red[32];
  pdl_launch();
  const int t = blockIdx.x;
  const int pos = positions[t], seq = seq_of_token[t];
  const int nq = p.n_heads * p.hd, nk = p.n_kv * p.hd, nv = p.v_mode == 0 ? p.n_kv * p.vd : 0;
  const int half = p.rot >> 1, vhalf = p.vinv_f || p.vinv_d ? p.vd >> 1 : 0;
  float* cs = qs + nq + nk + nv;      // [half] cos, [half] sin
  float* vcs = cs + 2 * half;         // [vhalf] cos, [vhalf] sin
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float c, s;
    rotary_cs(pos, j, p.inv_f, p.inv_d, c, s);
    cs[j] = c * p.magnitude;
    cs[half + j] = s * p.magnitude;
  }
  for (int j = threadIdx.x; j < vhalf; j += blockDim.x) rotary_cs(pos, j, p.vinv_f, p.vinv_d, vcs[j], vcs[vhalf + j]);
  pdl_wait();
  const TP* row = proj + (long long)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq + nk + nv; i += blockDim.x) {
    float v = to_f32<TP>(row[i]);
    if (p.bias) v += p.bias[i];
    qs[i] = v;
    if (i < nq) sq = fmaf(v, v, sq);
    else if (i < nq + nk) sk = fmaf(v, v, sk);
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  __syncthreads();
  const float iq = p.q_w ? 1.0f / sqrtf(sq / (float)nq + p.eps) : 1.0f;
  const float ik = p.k_w ? 1.0f / sqrtf(sk / (float)nk + p.eps) : 1.0f;
  // queries and keys: `half` pairs and hd - rot channels that pass, per head
  const int per_head = p.hd - half;
  const int heads = p.n_heads + (write_kv ? p.n_kv : 0);
  for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, j = idx - h * per_head;
    const bool is_k = h >= p.n_heads;
    const int base = h * p.hd;                  // the keys follow the queries in the row
    const float* w = is_k ? p.k_w : p.q_w;
    const int wb = is_k ? base - nq : base;
    const float inv = is_k ? ik : iq;
    const long long off = is_k ? paged_offset(pk, seq, pos, h - p.n_heads) : 0;
    T* dst = is_k ? k_pool + off : q_out + (long long)t * nq + base;
    if (j < half) {
      const int a = j, b = j + half;
      const float u = qs[base + a] * inv * (w ? w[wb + a] : 1.0f), v = qs[base + b] * inv * (w ? w[wb + b] : 1.0f);
      const float c = cs[j], s = cs[half + j];
      dst[a] = from_f32<T>(u * c - v * s);
      dst[b] = from_f32<T>(v * c + u * s);
    } else {
      const int ch = p.rot + (j - half);
      dst[ch] = from_f32<T>(qs[base + ch] * inv * (w ? w[wb + ch] : 1.0f));
    }
  }
  if (!write_kv) return;
  // values
  const int vper = p.vd - vhalf;
  const float* vsrc = p.v_mode == 0 ? qs + nq + nk : qs + nq;       // own values, or the keys as projected
  const int vstride = p.v_mode == 0 ? p.vd : p.hd;
  for (int idx = threadIdx.x; idx < p.n_kv * vper; idx += blockDim.x) {
    const int h = idx / vper, j = idx - h * vper;
    const float* src = vsrc + h * vstride;
    T* dst = v_pool + paged_offset(pvv, seq, pos, h);
    if (j < vhalf) {
      const float u = src[j], v = src[j + vhalf];
      const float c = vcs[j], s = vcs[vhalf + j];
      dst[j] = from_f32<T>(u * c - v * s);
      dst[j + vhalf] = from_f32<T>(v * c + u * s);
    } else {
      const int ch = 2 * vhalf + (j - vhalf);
      dst[ch] = from_f32<T>(src[ch]);
    }
  }
}

MF_API int mf_qk_norm_rope(const void* proj, int ld, int dtype, int out_dtype, int T, int n_heads, int n_kv, int hd, int vd, int rot,
                           int v_mode, float eps, float magnitude, const float* bias, const float* q_w,
                           const float* k_w, const float* inv_f, const double* inv_d, const float* vinv_f,
                           const double* vinv_d, const int* positions, const int* seq_of_token,
                           const int* block_table, int bt_stride, int page_size, void* q_out, void* k_pool,
                           void* v_pool, int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1) || (rot > 0 && !inv_f && !inv_d)) return MF_ERR_BAD_ARG;
  if (v_mode < 0 || v_mode > 1 || (v_mode == 1 && vd != hd) || vd <= 0) return MF_ERR_BAD_ARG;
  const bool vrot = vinv_f || vinv_d;
  if (vrot && (vd & 1)) return MF_ERR_BAD_ARG;
  const QkPrepare p{n_heads, n_kv, hd, vd, rot, v_mode, eps, magnitude, bias, q_w, k_w, inv_f, inv_d, vinv_f, vinv_d};
  const PagedView pk{block_table, bt_stride, page_size, n_kv, hd};
  const PagedView pvv{block_table, bt_stride, page_size, n_kv, vd};
  const int n = n_heads * hd + n_kv * hd + (v_mode == 0 ? n_kv * vd : 0);
  const size_t smem = (size_t)(n + rot + (vrot ? vd : 0) + 4) * sizeof(float);
  if (smem > 200 * 1024) return MF_ERR_BAD_ARG;
  mf_count(MF_K_QK_NORM_ROPE);
#define QK_LAUNCH(TP, TT)                                                                                          \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(qk_norm_rope_kernel<TP, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    return (int)launch_dep(qk_norm_rope_kernel<TP, TT>, dim3(T), dim3(256), smem, stream, (const TP*)proj, ld, p,  \
                           positions, seq_of_token, pk, pvv, (TT*)q_out, (TT*)k_pool, (TT*)v_pool, write_kv);      \
  } while (0)
  if (dtype == MF_F32 && out_dtype == MF_F32) QK_LAUNCH(float, float);
  if (dtype == MF_F32 && out_dtype == MF_BF16) QK_LAUNCH(float, __nv_bfloat16);
  if (dtype == MF_BF16 && out_dtype == MF_BF16) QK_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef QK_LAUNCH
  return MF_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ heads of a row turned by the position
// x [T, n_heads * d] in place: pair (m, m + rot/2) of the first `rot` channels of every head by
// sign * position * inv[m].
template <typename T>
__global__ void __launch_bounds__(256)
rotate_rows_kernel(T* __restrict__ x, int n_heads, int d, int rot, const int* __restrict__ positions,
                   const float* __restrict__ inv_f, const double* __restrict__ inv_d, float sign) {
  extern __shared__ float rr_cs[];
  pdl_launch();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float c, s;
    rotary_cs(pos, j, inv_f, inv_d, c, s);
    rr_cs[j] = c;
    rr_cs[half + j] = sign * s;
  }
  __syncthreads();
  pdl_wait();
  T* row = x + (long long)t * n_heads * d;
  for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
    const int h = idx / half, j = idx - h * half;
    T* p = row + (long long)h * d;
    const float u = to_f32<T>(p[j]), v = to_f32<T>(p[j + half]);
    const float c = rr_cs[j], s = rr_cs[half + j];
    p[j] = from_f32<T>(u * c - v * s);
    p[j + half] = from_f32<T>(v * c + u * s);
  }
}

MF_API int mf_rotate_rows(void* x, int dtype, int T, int n_heads, int d, int rot, const int* positions,
                          const float* inv_f, const double* inv_d, float sign, cudaStream_t stream) {
  if (T <= 0 || rot == 0) return 0;
  if (rot < 0 || rot > d || (rot & 1) || (!inv_f && !inv_d)) return MF_ERR_BAD_ARG;
  const size_t smem = (size_t)rot * sizeof(float);
  mf_count(MF_K_ROTATE_ROWS);
  if (dtype == MF_F32)
    return (int)launch_dep(rotate_rows_kernel<float>, dim3(T), dim3(256), smem, stream, (float*)x, n_heads, d, rot,
                           positions, inv_f, inv_d, sign);
  if (dtype == MF_BF16)
    return (int)launch_dep(rotate_rows_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, (__nv_bfloat16*)x,
                           n_heads, d, rot, positions, inv_f, inv_d, sign);
  return MF_ERR_BAD_DTYPE;
}
