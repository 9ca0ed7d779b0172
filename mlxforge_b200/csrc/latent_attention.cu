// Kernels around attention over a compressed latent: every token keeps one normed latent vector
// c [rank] and one rotated key part r [rot] that all heads share, `rank + rot` numbers in a cache
// lane of one key head.  With per-head expansions K_h = U_k,h c and V_h = U_v,h c the score of
// query (n_h | p_h) against a token is  n_h . (U_k,h c) + p_h . r  =  (U_k,h^T n_h) . c + p_h . r,
// so the attention runs over the latent itself: queries are (U_k,h^T n_h | p_h), `rank + rot`
// wide, keys are the cached rows, values their first `rank` channels, and the head's output is
// U_v,h applied to the attended latent.  Nothing is ever expanded per cached token.
//
//  * latent_prepare: one block per token over a row of projections [dq | dkv | ...]: the RMS norm
//    of the query latent (a model whose queries are projected directly has none: q_rank = 0), the
//    RMS norm of the key/value latent and the rotation of the shared key part, the last two
//    written into the token's place in the cache.
//  * latent_query: the rotated parts of the queries moved (rotated) behind the absorbed parts.
//  * head_linear: a product per head, out[t, h, :] = W_h x[t, h, :] with W [heads, N, K], rows
//    and heads of x and out at given strides, optionally times sigmoid(gate), the gate of output
//    n of head h read at gate[t * gate_ld + h * gate_hs + n * gate_ns] (one number per channel:
//    gate_hs = N, gate_ns = 1; one per head: gate_hs = 1, gate_ns = 0); accumulation in
//    32-bit, a warp per output element.  For few tokens; many tokens take the tensor-core one.
//
// The rotation takes its pairing (half-split or adjacent channels), how many of the `rot` channels
// turn (`rot_dims`, the rest pass unchanged) and a factor on cosine and sine (`mag`; 1 for the plain
// rotation, the attention factor of a stretched frequency table otherwise) as arguments.
#include "rotary.cuh"

// dst[0 .. rot) = rotation of src[0 .. rot): the first rot_dims channels turn in pairs, the rest are copied
template <typename T>
__device__ __forceinline__ void rotate_part(const T* __restrict__ src, T* __restrict__ dst, int rot, int rot_dims,
                                            int layout, float mag, int pos, const float* __restrict__ inv_f,
                                            const double* __restrict__ inv_d, int first, int step) {
  const int half = rot_dims >> 1;
  for (int j = first; j < half; j += step) {
    float c, s;
    rotary_cs(pos, j, inv_f, inv_d, c, s);
    c *= mag;
    s *= mag;
    int a, b;
    rotary_pair(layout, rot_dims, j, a, b);
    const float u = to_f32<T>(src[a]), v = to_f32<T>(src[b]);
    dst[a] = from_f32<T>(u * c - v * s);
    dst[b] = from_f32<T>(v * c + u * s);
  }
  for (int i = rot_dims + first; i < rot; i += step) dst[i] = src[i];
}

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, int ld, int q_rank, int kv_off, int rank, int rot,
                                      const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                      PagedView pv, const float* __restrict__ inv_f, const double* __restrict__ inv_d,
                                      T* __restrict__ cq_out, T* __restrict__ k_pool, int write_kv, int layout,
                                      int rot_dims, float mag) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = proj + (long long)t * ld;
  if (q_rank > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
      const float v = to_f32<T>(row[i]);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
    T* o = cq_out + (long long)t * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) o[i] = from_f32<T>(to_f32<T>(row[i]) * inv * wq[i]);
  }
  if (!write_kv) return;
  const int pos = positions[t], seq = seq_of_token[t];
  const T* kv = row + kv_off;
  T* dst = k_pool + paged_offset(pv, seq, pos, 0);
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f32<T>(kv[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(kv[i]) * inv * wkv[i]);
  rotate_part<T>(kv + rank, dst + rank, rot, rot_dims, layout, mag, pos, inv_f, inv_d, threadIdx.x, blockDim.x);
}

MF_API int mf_latent_prepare(const void* proj, int dtype, int T, int ld, int q_rank, int kv_off, int rank, int rot,
                             const float* wq, const float* wkv, float eps, const int* positions,
                             const int* seq_of_token, const int* block_table, int bt_stride, int page_size,
                             const float* inv_f, const double* inv_d, void* cq_out, void* k_pool, int write_kv,
                             int layout, int rot_dims, float mag, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank < 0 || rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return MF_ERR_BAD_ARG;
  if (layout != MF_ROT_HALF && layout != MF_ROT_PAIRS) return MF_ERR_BAD_ARG;
  if (q_rank == 0 && !write_kv) return 0;
  PagedView pv{block_table, bt_stride, page_size, 1, rank + rot};
  mf_count(MF_K_LATENT_PREPARE);
  if (dtype == MF_F32)
    return (int)launch_dep(latent_prepare_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)proj, ld, q_rank,
                           kv_off, rank, rot, wq, wkv, eps, positions, seq_of_token, pv, inv_f, inv_d, (float*)cq_out,
                           (float*)k_pool, write_kv, layout, rot_dims, mag);
  if (dtype == MF_BF16)
    return (int)launch_dep(latent_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream,
                           (const __nv_bfloat16*)proj, ld, q_rank, kv_off, rank, rot, wq, wkv, eps, positions,
                           seq_of_token, pv, inv_f, inv_d, (__nv_bfloat16*)cq_out, (__nv_bfloat16*)k_pool, write_kv,
                           layout, rot_dims, mag);
  return MF_ERR_BAD_DTYPE;
}

// q [T, heads, dim + rot] in rows q_ld apart -> q_full[t, h, rank : rank + rot] = rotation of q[t, h, dim : dim + rot]
template <typename T>
__global__ void latent_query_kernel(const T* __restrict__ q, long long q_ld, int n_heads, int dim, int rot, int rank,
                                    const int* __restrict__ positions, const float* __restrict__ inv_f,
                                    const double* __restrict__ inv_d, T* __restrict__ q_full, int layout, int rot_dims,
                                    float mag) {
  pdl_launch();
  const int t = blockIdx.x;
  const int pos = positions[t];
  pdl_wait();
  // a group of lanes per head: 32 where the block has room for all heads, else the heads take turns
  const int per = 32, groups = blockDim.x / per, g = threadIdx.x / per, l = threadIdx.x - g * per;
  for (int h = g; h < n_heads; h += groups) {
    const T* src = q + t * q_ld + (long long)h * (dim + rot) + dim;
    T* dst = q_full + ((long long)t * n_heads + h) * (rank + rot) + rank;
    rotate_part<T>(src, dst, rot, rot_dims, layout, mag, pos, inv_f, inv_d, l, per);
  }
}

MF_API int mf_latent_query(const void* q, long long q_ld, int dtype, int T, int n_heads, int dim, int rot, int rank,
                           const int* positions, const float* inv_f, const double* inv_d, void* q_full, int layout,
                           int rot_dims, float mag, cudaStream_t stream) {
  if (T <= 0 || rot == 0) return 0;
  if (rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return MF_ERR_BAD_ARG;
  if (layout != MF_ROT_HALF && layout != MF_ROT_PAIRS) return MF_ERR_BAD_ARG;
  mf_count(MF_K_LATENT_QUERY);
  if (dtype == MF_F32)
    return (int)launch_dep(latent_query_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)q, q_ld, n_heads,
                           dim, rot, rank, positions, inv_f, inv_d, (float*)q_full, layout, rot_dims, mag);
  if (dtype == MF_BF16)
    return (int)launch_dep(latent_query_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)q,
                           q_ld, n_heads, dim, rot, rank, positions, inv_f, inv_d, (__nv_bfloat16*)q_full, layout,
                           rot_dims, mag);
  return MF_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------------------- a product per head
constexpr int HL_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(HL_WARPS * 32)
head_linear_kernel(const T* __restrict__ x, long long x_ld, int x_hs, const T* __restrict__ w, T* __restrict__ out,
                   long long out_ld, int out_hs, int N, int K, const T* __restrict__ gate, long long gate_ld, int gate_hs,
                   int gate_ns) {
  extern __shared__ float xs[];          // [K]
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const T* xr = x + t * x_ld + (long long)h * x_hs;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f32<T>(xr[k]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* wh = w + (long long)h * N * K;
  T* orow = out + t * out_ld + (long long)h * out_hs;
  const T* grow = gate ? gate + t * gate_ld + (long long)h * gate_hs : nullptr;
  for (int n = warp; n < N; n += HL_WARPS) {
    const T* wr = wh + (long long)n * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], to_f32<T>(wr[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      if (grow) acc *= 1.0f / (1.0f + expf(-to_f32<T>(grow[n * gate_ns])));
      orow[n] = from_f32<T>(acc);
    }
  }
}

// ---------------------------------------------------------------------------- the same on tensor cores
// bfloat16, many tokens: a block per (64 tokens, head, 64 outputs).  The head's rows of x and of W
// (both K wide, K a multiple of 16) are staged whole in shared memory, each of the four warps owns
// 16 tokens and all 64 outputs: mma.sync m16n8k16 over K, 32-bit accumulators, the gate in the
// epilogue.  The order of a sum depends on K alone, so a token's result does not depend on the batch.
namespace {
constexpr int HM_BM = 64, HM_BN = 64, HM_WARPS = 4;

__device__ __forceinline__ void hm_cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void hm_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void hm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
}  // namespace

__global__ void __launch_bounds__(HM_WARPS * 32)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int x_hs, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ out, long long out_ld, int out_hs, int T, int N, int K,
                       const __nv_bfloat16* __restrict__ gate, long long gate_ld, int gate_hs, int gate_ns) {
  extern __shared__ __align__(16) unsigned char hm_smem[];
  const int ld = K + 8, chunks = K >> 3;
  __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(hm_smem);      // [HM_BM][ld]
  __nv_bfloat16* w_s = x_s + HM_BM * ld;                                // [HM_BN][ld]
  const int t0 = blockIdx.x * HM_BM, h = blockIdx.y, n0 = blockIdx.z * HM_BN;
  const __nv_bfloat16* wh = w + ((long long)h * N + n0) * K;
  for (int i = threadIdx.x; i < HM_BN * chunks; i += HM_WARPS * 32) {      // the weights never change: before the wait
    const int r = i / chunks, c = i - r * chunks;
    hm_cp_async_16(w_s + r * ld + c * 8, wh + (long long)min(r, N - n0 - 1) * K + c * 8, n0 + r < N);
  }
  pdl_launch();
  pdl_wait();
  for (int i = threadIdx.x; i < HM_BM * chunks; i += HM_WARPS * 32) {
    const int r = i / chunks, c = i - r * chunks;
    const int t = min(t0 + r, T - 1);
    hm_cp_async_16(x_s + r * ld + c * 8, x + t * x_ld + (long long)h * x_hs + c * 8, t0 + r < T);
  }
  asm volatile("cp.async.commit_group;\n" ::: "memory");
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  float acc[HM_BN / 8][4];
#pragma unroll
  for (int j = 0; j < HM_BN / 8; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  for (int kk = 0; kk < K; kk += 16) {
    unsigned a[4];
    hm_ldmatrix_x4(a, x_s + (warp * 16 + (lane & 15)) * ld + kk + (lane >> 4) * 8);
#pragma unroll
    for (int j = 0; j < HM_BN / 8; j += 2) {
      unsigned b[4];
      const int mi = lane >> 3, r = lane & 7;
      hm_ldmatrix_x4(b, w_s + (j * 8 + (mi >> 1) * 8 + r) * ld + kk + (mi & 1) * 8);
      hm_mma(acc[j], a, b[0], b[1]);
      hm_mma(acc[j + 1], a, b[2], b[3]);
    }
  }
#pragma unroll
  for (int hh = 0; hh < 2; hh++) {
    const int t = t0 + warp * 16 + g + hh * 8;
    if (t >= T) continue;
    __nv_bfloat16* orow = out + t * out_ld + (long long)h * out_hs;
    const __nv_bfloat16* grow = gate ? gate + t * gate_ld + (long long)h * gate_hs : nullptr;
#pragma unroll
    for (int j = 0; j < HM_BN / 8; j++) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int n = n0 + j * 8 + tq * 2 + e;
        if (n < N) {
          float v = acc[j][hh * 2 + e];
          if (grow) v *= 1.0f / (1.0f + __expf(-__bfloat162float(grow[n * gate_ns])));
          orow[n] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

// Whether the tensor-core kernel takes these operands: K a multiple of 16 that fits shared memory,
// rows and heads of x starting on 16-byte boundaries.
MF_API int mf_head_linear_mma_ok(long long x_ld, int x_hs, int K) {
  return (K % 16 == 0 && K <= 512 && x_ld % 8 == 0 && x_hs % 8 == 0) ? 1 : 0;
}

MF_API int mf_head_linear_mma(const void* x, long long x_ld, int x_hs, const void* w, void* out, long long out_ld,
                              int out_hs, int T, int n_heads, int N, int K, const void* gate, long long gate_ld,
                              int gate_hs, int gate_ns, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!mf_head_linear_mma_ok(x_ld, x_hs, K) || n_heads <= 0 || n_heads > 65535 || N <= 0) return MF_ERR_BAD_ARG;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return MF_ERR_BAD_ARG;
  const size_t smem = (size_t)(HM_BM + HM_BN) * (K + 8) * sizeof(__nv_bfloat16);
  static DeviceOnce once;
  const int dev = mf_current_device();
  if (dev < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(head_linear_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return (int)e;
    once.done[dev] = true;
  }
  mf_count(MF_K_HEAD_LINEAR_MMA);
  dim3 grid((T + HM_BM - 1) / HM_BM, n_heads, (N + HM_BN - 1) / HM_BN);
  return (int)launch_dep(head_linear_mma_kernel, grid, dim3(HM_WARPS * 32), smem, stream, (const __nv_bfloat16*)x, x_ld,
                         x_hs, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_ld, out_hs, T, N, K,
                         (const __nv_bfloat16*)gate, gate_ld, gate_hs, gate_ns);
}

MF_API int mf_head_linear(const void* x, long long x_ld, int x_hs, const void* w, void* out, long long out_ld,
                          int out_hs, int dtype, int T, int n_heads, int N, int K, const void* gate,
                          long long gate_ld, int gate_hs, int gate_ns, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_heads <= 0 || n_heads > 65535 || N <= 0 || K <= 0 || K > 8192) return MF_ERR_BAD_ARG;
  const size_t smem = (size_t)K * sizeof(float);
  mf_count(MF_K_HEAD_LINEAR);
  if (dtype == MF_F32)
    return (int)launch_dep(head_linear_kernel<float>, dim3(T, n_heads), dim3(HL_WARPS * 32), smem, stream,
                           (const float*)x, x_ld, x_hs, (const float*)w, (float*)out, out_ld, out_hs, N, K,
                           (const float*)gate, gate_ld, gate_hs, gate_ns);
  if (dtype == MF_BF16)
    return (int)launch_dep(head_linear_kernel<__nv_bfloat16>, dim3(T, n_heads), dim3(HL_WARPS * 32), smem, stream,
                           (const __nv_bfloat16*)x, x_ld, x_hs, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_ld,
                           out_hs, N, K, (const __nv_bfloat16*)gate, gate_ld, gate_hs, gate_ns);
  return MF_ERR_BAD_DTYPE;
}
