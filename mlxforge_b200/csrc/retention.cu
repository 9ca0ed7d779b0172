// Retention: linear attention with a fixed decay per head and no softmax.  Per head, with a
// 32-bit state S [dim, vdim] per request that starts at zero:
//
//     S_t = decay_h S_(t-1) + k_t v_t^T ,     o_t = S_t^T q_t
//
// q and k are rotated by position (half-split pairs over the first `rot` channels), k is then
// multiplied by `k_scale`; each head's o_t is divided by its root mean square (no weight),
// multiplied by silu(gate) and handed to the output projection.
//
//  * retention_prepare: one block per token; rotation and key scaling into 32-bit [T, 2 heads dim].
//  * retention_recurrence: every column of S is independent, so the recurrence is parallel over
//    (sequence, head, column) and serial in time only.  Eight lanes share a column and hold
//    dim/8 of its rows in registers; q and k of the coming tokens are staged in shared memory,
//    eight tokens at a time.  A step continues from the slot's state, so the result does not
//    depend on how a prompt was cut.
//  * retention_output: per token and head the read-out (summed over the row groups that a staged
//    launch spreads a head's state over) over its root mean square, times silu(gate).
#include "rotary.cuh"

namespace {
constexpr int RT_LANES = 8;                 // lanes that share one column of S
constexpr int RT_COLS = 16;                 // columns per block
constexpr int RT_THREADS = RT_LANES * RT_COLS;
constexpr int RT_CHUNK = 8;                 // tokens staged at a time
}  // namespace

// act 1: SiLU of every query and key channel before anything else.  v_out (optional): the row's `nv`
// channels from column `v_off` on, through the same activation, in 32-bit [T, nv].
template <typename T>
__global__ void retention_prepare_kernel(const T* __restrict__ proj, int ld, int n_heads, int dim, int rot,
                                         float k_scale, const int* __restrict__ positions,
                                         const float* __restrict__ inv_f, const double* __restrict__ inv_d,
                                         float* __restrict__ qk, int act, float* __restrict__ v_out, int v_off, int nv) {
  extern __shared__ float cs[];            // [half] cos, [half] sin
  pdl_launch();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) rotary_cs(pos, j, inv_f, inv_d, cs[j], cs[half + j]);
  __syncthreads();
  pdl_wait();
  const T* row = proj + (long long)t * ld;
  float* out = qk + (long long)t * 2 * n_heads * dim;
  const int per_head = dim - half;
  auto rd = [&](const T* p) {
    const float x = to_f32<T>(*p);
    return act ? x / (1.0f + expf(-x)) : x;
  };
  for (int idx = threadIdx.x; idx < 2 * n_heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, j = idx - h * per_head;       // heads 0..n-1: queries, n..2n-1: keys
    const T* src = row + (long long)h * dim;
    float* dst = out + (long long)h * dim;
    const float f = h >= n_heads ? k_scale : 1.0f;
    if (j < half) {
      const float c = cs[j], s = cs[half + j];
      const float u = rd(src + j), v = rd(src + j + half);
      dst[j] = (u * c - v * s) * f;
      dst[j + half] = (v * c + u * s) * f;
    } else {
      const int ch = rot + (j - half);
      dst[ch] = rd(src + ch) * f;
    }
  }
  if (v_out)
    for (int i = threadIdx.x; i < nv; i += blockDim.x) v_out[(long long)t * nv + i] = rd(row + v_off + i);
}

MF_API int mf_retention_prepare(const void* proj, int dtype, int T, int ld, int n_heads, int dim, int rot,
                                float k_scale, const int* positions, const float* inv_f, const double* inv_d,
                                float* qk, int act, float* v_out, int v_off, int nv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > dim || (rot & 1) || (rot > 0 && !inv_f && !inv_d)) return MF_ERR_BAD_ARG;
  const size_t smem = (size_t)(rot > 0 ? rot : 1) * sizeof(float);
  mf_count(MF_K_RETENTION_PREPARE);
  if (dtype == MF_F32)
    return (int)launch_dep(retention_prepare_kernel<float>, dim3(T), dim3(256), smem, stream, (const float*)proj, ld,
                           n_heads, dim, rot, k_scale, positions, inv_f, inv_d, qk, act, v_out, v_off, nv);
  if (dtype == MF_BF16)
    return (int)launch_dep(retention_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream,
                           (const __nv_bfloat16*)proj, ld, n_heads, dim, rot, k_scale, positions, inv_f, inv_d, qk,
                           act, v_out, v_off, nv);
  return MF_ERR_BAD_DTYPE;
}

// qk [T, 2 heads dim] (32-bit, prepared); v read from the projections' rows (v + t * v_ld + h * vdim).
// state [slots, heads, dim, vdim] with `state_stride` floats per slot.  o_out [T, heads * vdim] 32-bit.
template <typename T, int RPL>
__global__ void __launch_bounds__(RT_THREADS)
retention_recurrence_kernel(const float* __restrict__ qk, const T* __restrict__ v, long long v_ld,
                            const float* __restrict__ decay, float* __restrict__ state, long long state_stride,
                            const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                            const int* __restrict__ slots, float* __restrict__ o_out, int n_heads, int dim, int vdim) {
  extern __shared__ float sm[];            // [RT_CHUNK][2 dim] q then k of a token, [RT_CHUNK][RT_COLS] v
  float* v_s = sm + RT_CHUNK * 2 * dim;
  pdl_launch();
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * RT_COLS;
  const int lane = threadIdx.x % RT_LANES, cl = threadIdx.x / RT_LANES;
  const int c = c0 + cl;
  const bool col_ok = c < vdim;
  const int t0 = seq_q_start[s], n = seq_q_len[s];
  const float g = decay[h];
  float* S = state + (long long)slots[s] * state_stride + (long long)h * dim * vdim;
  float st[RPL];
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int r = lane + i * RT_LANES;
    st[i] = (col_ok && r < dim) ? S[(long long)r * vdim + c] : 0.f;
  }
  for (int b = 0; b < n; b += RT_CHUNK) {
    const int nb = min(RT_CHUNK, n - b);
    __syncthreads();
    for (int i = threadIdx.x; i < nb * 2 * dim; i += RT_THREADS) {
      const int tt = i / (2 * dim), d = i - tt * 2 * dim;
      const int hh = d / dim, ch = d - hh * dim;         // 0: q, 1: k
      sm[i] = qk[(long long)(t0 + b + tt) * 2 * n_heads * dim + (long long)(hh * n_heads + h) * dim + ch];
    }
    for (int i = threadIdx.x; i < nb * RT_COLS; i += RT_THREADS) {
      const int tt = i / RT_COLS, cc = i - tt * RT_COLS;
      v_s[i] = (c0 + cc < vdim) ? to_f32<T>(v[(long long)(t0 + b + tt) * v_ld + (long long)h * vdim + c0 + cc]) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nb; tt++) {
      const float* qs = sm + tt * 2 * dim;
      const float* ks = qs + dim;
      const float vc = v_s[tt * RT_COLS + cl];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i++) {
        const int r = lane + i * RT_LANES;
        if (r < dim) {
          st[i] = fmaf(g, st[i], ks[r] * vc);
          acc = fmaf(st[i], qs[r], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (lane == 0 && col_ok) o_out[(long long)(t0 + b + tt) * n_heads * vdim + (long long)h * vdim + c] = acc;
    }
  }
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int r = lane + i * RT_LANES;
    if (col_ok && r < dim) S[(long long)r * vdim + c] = st[i];
  }
}

// ---------------------------------------------------------------------------- the same, staged
// For sizes in whole pieces (dim a multiple of the rows per block, vdim of 16, 16-byte aligned rows): a block owns
// RS_ROWS rows x RT_COLS columns of S, so that a head's state is spread over dim/RS_ROWS x vdim/RT_COLS
// blocks (an element of S depends on no other element; only the read-out sums over rows, and that sum
// is finished by the output kernel over the row groups' partial read-outs).  The block's share of q, k
// and v of the coming tokens arrives through a ring of cp.async stages, RS_CHUNK tokens each, so that no
// token waits for memory.
namespace {
constexpr int RS_CHUNK = 16;
constexpr int RS_STAGES = 4;

__device__ __forceinline__ void rs_cp_async_16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
}  // namespace

template <typename T, int RS_ROWS>
__global__ void __launch_bounds__(RT_THREADS)
retention_recurrence_staged_kernel(const float* __restrict__ qk, const T* __restrict__ v, long long v_ld,
                                   const float* __restrict__ decay, float* __restrict__ state, long long state_stride,
                                   const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                                   const int* __restrict__ slots, float* __restrict__ o_part, long long part_stride,
                                   int n_heads, int dim, int vdim) {
  constexpr int RS_RPL = RS_ROWS / RT_LANES;
  constexpr int V_PIECES = RT_COLS * sizeof(T) / 16;               // 16-byte pieces of a token's values
  constexpr int PIECES = 2 * RS_ROWS / 4 + V_PIECES;               // q, k, v of one token
  constexpr int TOKEN_FLOATS = 2 * RS_ROWS + RT_COLS * sizeof(T) / 4;
  __shared__ __align__(16) float ring[RS_STAGES][RS_CHUNK][TOKEN_FLOATS];
  pdl_launch();
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y;
  const int n_cb = vdim / RT_COLS;
  const int rg = blockIdx.z / n_cb, c0 = (blockIdx.z - rg * n_cb) * RT_COLS, r0 = rg * RS_ROWS;
  const int lane = threadIdx.x % RT_LANES, cl = threadIdx.x / RT_LANES;
  const int t0 = seq_q_start[s], n = seq_q_len[s];
  const float g = decay[h];
  float* S = state + (long long)slots[s] * state_stride + ((long long)h * dim + r0) * vdim + c0 + cl;
  float st[RS_RPL];
#pragma unroll
  for (int i = 0; i < RS_RPL; i++) st[i] = S[(long long)(lane + i * RT_LANES) * vdim];
  const int n_chunks = (n + RS_CHUNK - 1) / RS_CHUNK;

  auto fetch = [&](int chunk) {
    const int stage = chunk % RS_STAGES;
    const int nb = min(RS_CHUNK, n - chunk * RS_CHUNK);
    for (int i = threadIdx.x; i < nb * PIECES; i += RT_THREADS) {
      const int tt = i / PIECES, p = i - tt * PIECES;
      const long long t = t0 + chunk * RS_CHUNK + tt;
      float* dst = &ring[stage][tt][0] + p * 4;
      if (p < 2 * RS_ROWS / 4) {
        const int which = p / (RS_ROWS / 4), q4 = p - which * (RS_ROWS / 4);      // 0: q, 1: k
        rs_cp_async_16(dst, qk + t * 2 * n_heads * dim + (long long)(which * n_heads + h) * dim + r0 + q4 * 4);
      } else {
        const int v4 = p - 2 * RS_ROWS / 4;
        rs_cp_async_16(dst, reinterpret_cast<const char*>(v + t * v_ld + (long long)h * vdim + c0) + v4 * 16);
      }
    }
  };
#pragma unroll
  for (int c = 0; c < RS_STAGES - 1; c++) {
    if (c < n_chunks) fetch(c);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  float* o = o_part + (long long)rg * part_stride + (long long)h * vdim + c0 + cl;
  for (int chunk = 0; chunk < n_chunks; chunk++) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(RS_STAGES - 2) : "memory");
    __syncthreads();          // the chunk has landed for everyone, and everyone is done with the stage refilled next
    if (chunk + RS_STAGES - 1 < n_chunks) fetch(chunk + RS_STAGES - 1);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    const int stage = chunk % RS_STAGES;
    const int nb = min(RS_CHUNK, n - chunk * RS_CHUNK);
    // four tokens at a time: only the state is a chain from token to token; the four read-outs' sums
    // over the lanes of a column go through their shuffles side by side
    for (int tt = 0; tt < nb; tt += 4) {
      float acc[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        acc[u] = 0.f;
        if (tt + u < nb) {
          const float* qs = &ring[stage][tt + u][0];
          const float* ks = qs + RS_ROWS;
          const float vc = to_f32<T>(reinterpret_cast<const T*>(ks + RS_ROWS)[cl]);
#pragma unroll
          for (int i = 0; i < RS_RPL; i++) {
            const int r = lane + i * RT_LANES;
            st[i] = fmaf(g, st[i], ks[r] * vc);
            acc[u] = fmaf(st[i], qs[r], acc[u]);
          }
        }
      }
#pragma unroll
      for (int m = 1; m < RT_LANES; m <<= 1)
#pragma unroll
        for (int u = 0; u < 4; u++) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], m);
      if (lane == 0) {
#pragma unroll
        for (int u = 0; u < 4; u++)
          if (tt + u < nb) o[(long long)(t0 + chunk * RS_CHUNK + tt + u) * n_heads * vdim] = acc[u];
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < RS_RPL; i++) S[(long long)(lane + i * RT_LANES) * vdim] = st[i];
}

// Rows of S per block of the staged kernel: 16, 32 or 64.  Fewer rows spread a head over more blocks,
// more rows give a thread more of S to work on per operand it fetches.
static int g_retention_rows = 32;
MF_API int mf_set_retention_rows(int rows) {
  if (rows != 16 && rows != 32 && rows != 64) return MF_ERR_BAD_ARG;
  g_retention_rows = rows;
  return 0;
}

// How many partial read-outs (row groups) a launch writes: retention_output sums them.
MF_API int mf_retention_parts(int dim, int vdim, int v_dtype, long long v_ld) {
  const int vb = v_dtype == MF_F32 ? 4 : 2;
  const bool staged = dim % g_retention_rows == 0 && vdim % RT_COLS == 0 && (v_ld * vb) % 16 == 0 &&
                      (vdim * vb) % 16 == 0;
  return staged ? dim / g_retention_rows : 1;
}

template <typename T, int ROWS>
static int launch_staged(const float* qk, const void* v, long long v_ld, const float* decay, float* state,
                         long long state_stride, const int* seq_q_start, const int* seq_q_len, const int* slots,
                         float* o_out, long long part_stride, int n_seqs, int n_heads, int dim, int vdim,
                         cudaStream_t stream) {
  dim3 grid(n_seqs, n_heads, (dim / ROWS) * (vdim / RT_COLS));
  return (int)launch_dep(retention_recurrence_staged_kernel<T, ROWS>, grid, dim3(RT_THREADS), 0, stream, qk, (const T*)v,
                         v_ld, decay, state, state_stride, seq_q_start, seq_q_len, slots, o_out, part_stride, n_heads,
                         dim, vdim);
}

MF_API int mf_retention_recurrence(const float* qk, const void* v, int v_dtype, long long v_ld, const float* decay,
                                   float* state, long long state_stride, const int* seq_q_start,
                                   const int* seq_q_len, const int* slots, float* o_out, long long part_stride,
                                   int n_seqs, int n_heads, int dim, int vdim, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (dim <= 0 || dim > 64 * RT_LANES || vdim <= 0 || n_heads <= 0 || n_heads > 65535) return MF_ERR_BAD_ARG;
  // o_out holds mf_retention_parts(...) partial read-outs, `part_stride` floats apart
  if (mf_retention_parts(dim, vdim, v_dtype, v_ld) > 1 && ((uintptr_t)qk & 15) == 0 && ((uintptr_t)v & 15) == 0 &&
      (v_dtype == MF_F32 || v_dtype == MF_BF16)) {
    mf_count(MF_K_RETENTION_RECURRENCE);
#define RS_GO(TT, ROWS)                                                                                             \
  return launch_staged<TT, ROWS>(qk, v, v_ld, decay, state, state_stride, seq_q_start, seq_q_len, slots, o_out,     \
                                 part_stride, n_seqs, n_heads, dim, vdim, stream)
#define RS_ROWS_PICK(TT)                  \
  if (g_retention_rows == 16) RS_GO(TT, 16); \
  if (g_retention_rows == 32) RS_GO(TT, 32); \
  RS_GO(TT, 64)
    if (v_dtype == MF_F32) { RS_ROWS_PICK(float); }
    RS_ROWS_PICK(__nv_bfloat16);
#undef RS_ROWS_PICK
#undef RS_GO
  }
  if (mf_retention_parts(dim, vdim, v_dtype, v_ld) > 1) return MF_ERR_BAD_ARG;     // the caller sized o_out for parts
  dim3 grid(n_seqs, n_heads, (vdim + RT_COLS - 1) / RT_COLS);
  const size_t smem = (size_t)RT_CHUNK * (2 * dim + RT_COLS) * sizeof(float);
  const int per = (dim + RT_LANES - 1) / RT_LANES;
  mf_count(MF_K_RETENTION_RECURRENCE);
#define RT_LAUNCH(TT, RPL)                                                                                       \
  return (int)launch_dep(retention_recurrence_kernel<TT, RPL>, grid, dim3(RT_THREADS), smem, stream, qk,         \
                         (const TT*)v, v_ld, decay, state, state_stride, seq_q_start, seq_q_len, slots, o_out,   \
                         n_heads, dim, vdim)
#define RT_PICK(TT)              \
  if (per <= 4) RT_LAUNCH(TT, 4);  \
  if (per <= 8) RT_LAUNCH(TT, 8);  \
  if (per <= 16) RT_LAUNCH(TT, 16); \
  if (per <= 32) RT_LAUNCH(TT, 32); \
  RT_LAUNCH(TT, 64)
  if (v_dtype == MF_F32) { RT_PICK(float); }
  if (v_dtype == MF_BF16) { RT_PICK(__nv_bfloat16); }
#undef RT_PICK
#undef RT_LAUNCH
  return MF_ERR_BAD_DTYPE;
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * silu(gate[t, h, :]); a warp per (token, head).
// whole: one root mean square over all heads of the token instead of one per head.  weight (optional):
// [n_heads * vdim], multiplied in.  gate_act 1: the gate passes a sigmoid instead of SiLU.
template <typename T>
__global__ void retention_output_kernel(const float* __restrict__ o, int n_parts, long long part_stride,
                                        const T* __restrict__ gate, long long gate_ld, float eps, T* __restrict__ out,
                                        int n_heads, int vdim, const float* __restrict__ weight, int whole,
                                        int gate_act) {
  extern __shared__ float ro_ss[];      // [n_heads] sums of squares
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  auto read = [&](const float* orow, int d) {
    // the read-out is the sum of the row groups' partial read-outs, added in their order
    float v = orow[d];
    for (int p = 1; p < n_parts; p++) v += orow[p * part_stride + d];
    return v;
  };
  for (int h = warp; h < n_heads; h += nw) {
    const float* orow = o + ((long long)t * n_heads + h) * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) {
      const float v = read(orow, d);
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) ro_ss[h] = ss;
  }
  __syncthreads();
  float all = 0.f;
  if (whole)
    for (int h = 0; h < n_heads; h++) all += ro_ss[h];
  for (int h = warp; h < n_heads; h += nw) {
    const float* orow = o + ((long long)t * n_heads + h) * vdim;
    const T* grow = gate + (long long)t * gate_ld + (long long)h * vdim;
    const float inv = whole ? 1.0f / sqrtf(all / (float)(n_heads * vdim) + eps) : 1.0f / sqrtf(ro_ss[h] / (float)vdim + eps);
    T* dst = out + ((long long)t * n_heads + h) * vdim;
    for (int d = lane; d < vdim; d += 32) {
      const float g = to_f32<T>(grow[d]);
      const float sg = 1.0f / (1.0f + expf(-g));
      const float w = weight ? weight[h * vdim + d] : 1.0f;
      dst[d] = from_f32<T>(read(orow, d) * inv * w * (gate_act ? sg : g * sg));
    }
  }
}

MF_API int mf_retention_output(const float* o, int n_parts, long long part_stride, const void* gate, int dtype,
                               long long gate_ld, float eps, void* out, int T, int n_heads, int vdim,
                               const float* weight, int whole, int gate_act, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_parts < 1) return MF_ERR_BAD_ARG;
  mf_count(MF_K_RETENTION_OUTPUT);
  const int threads = n_heads >= 8 ? 256 : 32 * (n_heads > 0 ? n_heads : 1);
  const size_t smem = (size_t)(n_heads > 0 ? n_heads : 1) * sizeof(float);
  if (smem > 48 * 1024) return MF_ERR_BAD_ARG;
  if (dtype == MF_F32)
    return (int)launch_dep(retention_output_kernel<float>, dim3(T), dim3(threads), smem, stream, o, n_parts, part_stride,
                           (const float*)gate, gate_ld, eps, (float*)out, n_heads, vdim, weight, whole, gate_act);
  if (dtype == MF_BF16)
    return (int)launch_dep(retention_output_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, o, n_parts,
                           part_stride, (const __nv_bfloat16*)gate, gate_ld, eps, (__nv_bfloat16*)out, n_heads, vdim,
                           weight, whole, gate_act);
  return MF_ERR_BAD_DTYPE;
}
