// Causal GQA attention over the paged cache, any number of new tokens per
// sequence, float32 or bfloat16 storage, every score and the softmax in 32-bit.
// One block per (token, query head).  It is the attention of the 32-bit model
// path and the plain device reference the faster bfloat16 kernels are checked
// against.  Formula: src/model/sdpa.cpp:71-95 and src/model/decoder_model.cpp:260-275
// of hvasconcelos/mlxforge (scores * scale, causal mask aligned to the end of the
// keys, softmax over keys, p * v; query head h reads KV head h / (nh/nkv)).
//
// The query at position p of its sequence sees keys [lo, p], lo = 0 or
// p - window + 1 for a windowed lane.  Keys are visited in chunks of 128 starting
// at a multiple of 128, so the order of every sum depends only on the position.
#include "common.cuh"

#define CHUNK 128
#define MAX_ACC 4      // value channels per thread: values up to MAX_ACC * CHUNK wide

// Further options, all off at their defaults:
//  * keys and values of unlike width: a key row is pv.head_dim wide, a value row `vd`, and value
//    rows lie `v_ld` apart in their pool.  With v_pool == k_pool and v_ld == pv.head_dim the values
//    are the first `vd` channels of the keys (one latent per token that is key and value at once);
//  * keep_first > 0 (with a window): keys at positions below keep_first stay visible to every
//    later query, at their own positions;
//  * sink (one float per query head): exp(sink_h) joins the softmax denominator; it has no key
//    and no value and is not scaled;
//  * gate ([T, gate_ld], head h at column h * vd): the output is multiplied by sigmoid(gate).
template <typename T>
__global__ void __launch_bounds__(CHUNK)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, PagedView pv, int n_heads, float scale,
                         int window, int vd, int v_ld, int keep_first, const float* __restrict__ sink,
                         const T* __restrict__ gate, int gate_ld, float softcap) {
  extern __shared__ float smem[];
  float* qs = smem;                 // [hd]
  float* ps = smem + pv.head_dim;   // [CHUNK]
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y;
  const int hd = pv.head_dim;
  const int kvh = h / (n_heads / pv.n_kv_heads);
  const int pos = positions[t], seq = seq_of_token[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int keep = (window > 0 && keep_first > 0) ? min(keep_first, lo) : 0;   // kept keys before the window

  const T* qrow = q + ((long long)t * n_heads + h) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = to_f32<T>(qrow[d]);
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  if (sink) {                       // the sink as a key of score sink_h whose value is zero
    m = sink[h];
    l = 1.f;
  }
  float acc[MAX_ACC];
#pragma unroll
  for (int a = 0; a < MAX_ACC; a++) acc[a] = 0.f;
  const int first_win = (lo / CHUNK) * CHUNK;
  // the chunks of kept keys that lie wholly before the window's first chunk, then the window's
  for (int c0 = (keep > 0 ? 0 : first_win); c0 <= pos; c0 += CHUNK) {
    if (c0 < first_win && c0 >= keep) {
      c0 = first_win - CHUNK;
      continue;
    }
    const int j = c0 + threadIdx.x;
    float s = -INFINITY;
    if (j <= pos && (j >= lo || j < keep)) {
      const T* kr = k_pool + paged_offset(pv, seq, j, kvh);
      float dot = 0.f;
      for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    }
    const float cm = block_max(s, red);
    const float m_new = fmaxf(m, cm);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    __syncthreads();
    ps[threadIdx.x] = p;
    const float psum = block_sum(p, red);   // has __syncthreads inside: ps is visible after it
    l = l * alpha + psum;
    m = m_new;
#pragma unroll
    for (int a = 0; a < MAX_ACC; a++) acc[a] *= alpha;
    const int jn = min(CHUNK, pos - c0 + 1);
    for (int jj = 0; jj < jn; jj++) {
      const int key = c0 + jj;
      if (key < lo && key >= keep) continue;
      const float pj = ps[jj];
      const T* vr = v_pool + paged_offset(pv, seq, key, kvh) / hd * v_ld;
#pragma unroll
      for (int a = 0; a < MAX_ACC; a++)
        if ((int)threadIdx.x + a * CHUNK < vd) acc[a] = fmaf(pj, to_f32<T>(vr[threadIdx.x + a * CHUNK]), acc[a]);
    }
    __syncthreads();
  }
  T* orow = out + ((long long)t * n_heads + h) * vd;
  const T* grow = gate ? gate + (long long)t * gate_ld + (long long)h * vd : nullptr;
  const float inv = 1.0f / l;
#pragma unroll
  for (int a = 0; a < MAX_ACC; a++) {
    const int d = threadIdx.x + a * CHUNK;
    if (d < vd) {
      float o = acc[a] * inv;
      if (grow) o *= 1.0f / (1.0f + expf(-to_f32<T>(grow[d])));
      orow[d] = from_f32<T>(o);
    }
  }
}

static int launch_generic(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype, int T,
                          int n_heads, int n_kv, int hd, const int* positions, const int* seq_of_token,
                          const int* block_table, int bt_stride, int page_size, float scale, int window, int vd,
                          int v_ld, int keep_first, const float* sink, const void* gate, int gate_ld,
                          float softcap, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd > 1024 || vd <= 0 || vd > MAX_ACC * CHUNK || v_ld < vd || n_kv <= 0 || n_heads % n_kv)
    return MF_ERR_BAD_ARG;
  if (n_heads > 65535 || keep_first < 0) return MF_ERR_BAD_ARG;
  PagedView pv{block_table, bt_stride, page_size, n_kv, hd};
  dim3 grid(T, n_heads);
  const size_t smem = (size_t)(hd + CHUNK) * sizeof(float);
  if (dtype == MF_F32 || dtype == MF_BF16) mf_count(MF_K_ATTN_GENERIC);
  if (dtype == MF_F32)
    attention_generic_kernel<float><<<grid, CHUNK, smem, stream>>>(
        (const float*)q, (const float*)k_pool, (const float*)v_pool, (float*)out, positions, seq_of_token, pv,
        n_heads, scale, window, vd, v_ld, keep_first, sink, (const float*)gate, gate_ld, softcap);
  else if (dtype == MF_BF16)
    attention_generic_kernel<__nv_bfloat16><<<grid, CHUNK, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
        (__nv_bfloat16*)out, positions, seq_of_token, pv, n_heads, scale, window, vd, v_ld, keep_first, sink,
        (const __nv_bfloat16*)gate, gate_ld, softcap);
  else
    return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}

MF_API int mf_attention_generic(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                int T, int n_heads, int n_kv, int hd, const int* positions,
                                const int* seq_of_token, const int* block_table, int bt_stride,
                                int page_size, float scale, int window, cudaStream_t stream) {
  if (hd > 2 * CHUNK) return MF_ERR_BAD_ARG;
  return launch_generic(q, k_pool, v_pool, out, dtype, T, n_heads, n_kv, hd, positions, seq_of_token, block_table,
                        bt_stride, page_size, scale, window, hd, hd, 0, nullptr, nullptr, 0, 0.f, stream);
}

// The same with the options above: value width and row stride, kept first keys, sink, output gate.
MF_API int mf_attention_generic_ex(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                   int T, int n_heads, int n_kv, int hd, const int* positions,
                                   const int* seq_of_token, const int* block_table, int bt_stride,
                                   int page_size, float scale, int window, int vd, int v_ld, int keep_first,
                                   const float* sink, const void* gate, int gate_ld, float softcap,
                                   cudaStream_t stream) {
  return launch_generic(q, k_pool, v_pool, out, dtype, T, n_heads, n_kv, hd, positions, seq_of_token, block_table,
                        bt_stride, page_size, scale, window, vd, v_ld, keep_first, sink, gate, gate_ld, softcap, stream);
}
