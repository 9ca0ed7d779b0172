// What stands around a sublayer that reads the residual stream itself and is normalised on its way
// back into it:
//
//   h_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j)          (a causal convolution over time per channel,
//                                                            zeros before the sequence's start)
//   x_t <- x_t + rms(y_t) * g ,  y = s1 y1 + s2 y2           (RMS norm of the sublayer's output, or of the
//                                                            weighted sum of two branches' outputs)
//
// The stream x is 32-bit [T, H]; the convolution, the weighted sum, the norm and the add are 32-bit
// and h is rounded once.  The last taps-1 rows of x that a sequence's convolution has read are kept
// in the request's state slot ([taps-1, H] at `tail_off`), so a step goes on from where the step
// before ended however the tokens were cut; a second kernel moves them on after the first has read
// them.  Where every sequence of the step brings one token (decoding) a token's block is the only reader
// of its slot's rows and moves them on itself: one launch.
#include "common.cuh"

// ------------------------------------------------------------------ h = x + conv(x)
template <typename TO>
__global__ void __launch_bounds__(256)
conv_input_kernel(const float* __restrict__ x, int H, const float* __restrict__ w, int taps,
                  float* __restrict__ state, long long state_stride, long long tail_off,
                  const int* __restrict__ seq_of_token, const int* __restrict__ seq_q_start,
                  const int* __restrict__ slots, TO* __restrict__ out, int move_tail) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const int rel = t - seq_q_start[seq];
  float* tail = state + (long long)slots[seq] * state_stride + tail_off;      // [(taps-1), H]
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < taps; j++) {
      const int back = taps - 1 - j;
      const float v = rel - back >= 0 ? x[(long long)(t - back) * H + c] : tail[(long long)(rel - back + taps - 1) * H + c];
      a = fmaf(w[(long long)c * taps + j], v, a);
    }
    out[(long long)t * H + c] = from_f32<TO>(x[(long long)t * H + c] + a);
    if (move_tail)          // the sequence's only token: every row moves up one place, the token's row comes last
      for (int j = 0; j < taps - 1; j++)
        tail[(long long)j * H + c] = j < taps - 2 ? tail[(long long)(j + 1) * H + c] : x[(long long)t * H + c];
  }
}

// four channels a thread: 16-byte loads of x and of the tail (H a multiple of 4)
template <typename TO, int TAPS>
__global__ void __launch_bounds__(256)
conv_input_vec_kernel(const float* __restrict__ x, int H, const float* __restrict__ w,
                      float* __restrict__ state, long long state_stride, long long tail_off,
                      const int* __restrict__ seq_of_token, const int* __restrict__ seq_q_start,
                      const int* __restrict__ slots, TO* __restrict__ out, int move_tail) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const int rel = t - seq_q_start[seq];
  float* tail = state + (long long)slots[seq] * state_stride + tail_off;
  for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    float4 cur = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 seen[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; j++) {
      const int back = TAPS - 1 - j;
      const float4 v = rel - back >= 0 ? *reinterpret_cast<const float4*>(x + (long long)(t - back) * H + c)
                                       : *reinterpret_cast<const float4*>(tail + (long long)(rel - back + TAPS - 1) * H + c);
      seen[j] = v;
      if (back == 0) cur = v;
      a[0] = fmaf(w[(long long)(c + 0) * TAPS + j], v.x, a[0]);
      a[1] = fmaf(w[(long long)(c + 1) * TAPS + j], v.y, a[1]);
      a[2] = fmaf(w[(long long)(c + 2) * TAPS + j], v.z, a[2]);
      a[3] = fmaf(w[(long long)(c + 3) * TAPS + j], v.w, a[3]);
    }
    TO* o = out + (long long)t * H + c;
    o[0] = from_f32<TO>(cur.x + a[0]);
    o[1] = from_f32<TO>(cur.y + a[1]);
    o[2] = from_f32<TO>(cur.z + a[2]);
    o[3] = from_f32<TO>(cur.w + a[3]);
    if (move_tail) {        // the sequence's only token: what was read, one place on
#pragma unroll
      for (int j = 0; j < TAPS - 1; j++) *reinterpret_cast<float4*>(tail + (long long)j * H + c) = seen[j + 1];
    }
  }
}

// After the step the slot keeps the last taps-1 rows of x that the convolution has read.
__global__ void __launch_bounds__(256)
conv_input_tail_kernel(const float* __restrict__ x, int H, int taps, float* __restrict__ state, long long state_stride,
                       long long tail_off, const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                       const int* __restrict__ slots) {
  pdl_launch();
  pdl_wait();
  const int seq = blockIdx.x;
  const int start = seq_q_start[seq], n = seq_q_len[seq];
  float* tail = state + (long long)slots[seq] * state_stride + tail_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H; c += gridDim.y * blockDim.x) {
    for (int j = 0; j < taps - 1; j++) {          // ascending: a read is never behind a write
      const int src = n - (taps - 1) + j;
      tail[(long long)j * H + c] = src >= 0 ? x[(long long)(start + src) * H + c] : tail[(long long)(j + n) * H + c];
    }
  }
}

MF_API int mf_conv_input(const float* x, int T, int H, const float* w, int taps, float* state, long long state_stride,
                         long long tail_off, const int* seq_of_token, const int* seq_q_start, const int* seq_q_len,
                         const int* slots, int n_seqs, void* out, int out_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || H <= 0) return MF_ERR_BAD_ARG;
  if (out_dtype != MF_F32 && out_dtype != MF_BF16) return MF_ERR_BAD_DTYPE;
  mf_count(MF_K_CONV_INPUT);
  cudaError_t e;
  // one token from every sequence (the caller lays the step out so: T tokens of n_seqs sequences, none empty)
  const int single = (T == n_seqs && taps > 1) ? 1 : 0;
  const bool vec = H % 4 == 0 && tail_off % 4 == 0 && state_stride % 4 == 0 && ((uintptr_t)x & 15) == 0 &&
                   ((uintptr_t)state & 15) == 0 && taps >= 2 && taps <= 4;
  const int threads = vec ? (H / 4 >= 256 ? 256 : ((H / 4 + 31) / 32) * 32) : 256;
#define CI_VEC(TO, TAPS)                                                                                          \
  e = launch_dep(conv_input_vec_kernel<TO, TAPS>, dim3(T), dim3(threads), 0, stream, x, H, w, state, state_stride,  \
                 tail_off, seq_of_token, seq_q_start, slots, (TO*)out, single)
#define CI_ANY(TO)                                                                                                \
  do {                                                                                                            \
    if (vec && taps == 2) CI_VEC(TO, 2);                                                                          \
    else if (vec && taps == 3) CI_VEC(TO, 3);                                                                     \
    else if (vec && taps == 4) CI_VEC(TO, 4);                                                                     \
    else                                                                                                          \
      e = launch_dep(conv_input_kernel<TO>, dim3(T), dim3(256), 0, stream, x, H, w, taps, state, state_stride,    \
                     tail_off, seq_of_token, seq_q_start, slots, (TO*)out, single);                               \
  } while (0)
  if (out_dtype == MF_F32) CI_ANY(float);
  else CI_ANY(__nv_bfloat16);
#undef CI_ANY
#undef CI_VEC
  if (e != cudaSuccess) return (int)e;
  if (taps > 1 && !single) {
    const int by = (H + 1023) / 1024;
    e = launch_dep(conv_input_tail_kernel, dim3(n_seqs, by), dim3(256), 0, stream, x, H, taps, state, state_stride,
                   tail_off, seq_q_start, seq_q_len, slots);
  }
  return (int)e;
}

// ------------------------------------------------------------------ x += rms(s1 y1 + s2 y2) * g
// One block per token.  y1, y2 [T, H] in the dtype T1 (32-bit or bfloat16); y2 may be null.
template <typename T1>
__global__ void __launch_bounds__(256)
postnorm_add_kernel(float* __restrict__ x, int H, const T1* __restrict__ y1, float s1, const T1* __restrict__ y2,
                    float s2, const float* __restrict__ g, float eps) {
  extern __shared__ float pn_y[];      // [H]
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const long long t = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = s1 * to_f32<T1>(y1[t * H + c]);
    if (y2) v = fmaf(s2, to_f32<T1>(y2[t * H + c]), v);
    pn_y[c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) x[t * H + c] += pn_y[c] * inv * g[c];
}

// four channels a thread with 16-byte accesses to the stream (H a multiple of 4): the sums stay in registers
template <typename T1, int PER>
__global__ void __launch_bounds__(256)
postnorm_add_vec_kernel(float* __restrict__ x, int H, const T1* __restrict__ y1, float s1, const T1* __restrict__ y2,
                        float s2, const float* __restrict__ g, float eps) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const long long t = blockIdx.x;
  float y[PER][4];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PER; p++) {
    const int c = (p * 256 + threadIdx.x) * 4;
#pragma unroll
    for (int j = 0; j < 4; j++) y[p][j] = 0.f;
    if (c < H) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float v = s1 * to_f32<T1>(y1[t * H + c + j]);
        if (y2) v = fmaf(s2, to_f32<T1>(y2[t * H + c + j]), v);
        y[p][j] = v;
        ss = fmaf(v, v, ss);
      }
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int p = 0; p < PER; p++) {
    const int c = (p * 256 + threadIdx.x) * 4;
    if (c < H) {
      float4 xv = *reinterpret_cast<float4*>(x + t * H + c);
      const float4 gv = *reinterpret_cast<const float4*>(g + c);
      xv.x += y[p][0] * inv * gv.x;
      xv.y += y[p][1] * inv * gv.y;
      xv.z += y[p][2] * inv * gv.z;
      xv.w += y[p][3] * inv * gv.w;
      *reinterpret_cast<float4*>(x + t * H + c) = xv;
    }
  }
}

MF_API int mf_postnorm_add(float* x, int T, int H, const void* y1, float s1, const void* y2, float s2, int y_dtype,
                           const float* g, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)H * sizeof(float);
  if (H <= 0 || smem > 200 * 1024) return MF_ERR_BAD_ARG;
  mf_count(MF_K_POSTNORM_ADD);
  const bool vec = H % 4 == 0 && H <= 8 * 1024 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)g & 15) == 0;
#define PN_VEC(T1, PER)                                                                                           \
  return (int)launch_dep(postnorm_add_vec_kernel<T1, PER>, dim3(T), dim3(256), 0, stream, x, H, (const T1*)y1, s1, \
                         (const T1*)y2, s2, g, eps)
#define PN_LAUNCH(T1)                                                                                             \
  do {                                                                                                            \
    if (vec && H <= 1024) PN_VEC(T1, 1);                                                                          \
    if (vec && H <= 2048) PN_VEC(T1, 2);                                                                          \
    if (vec && H <= 4096) PN_VEC(T1, 4);                                                                          \
    if (vec) PN_VEC(T1, 8);                                                                                       \
    if (smem > 48 * 1024) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(postnorm_add_kernel<T1>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                           (int)smem);                                                            \
      if (e != cudaSuccess) return (int)e;                                                                        \
    }                                                                                                             \
    return (int)launch_dep(postnorm_add_kernel<T1>, dim3(T), dim3(256), smem, stream, x, H, (const T1*)y1, s1,    \
                           (const T1*)y2, s2, g, eps);                                                            \
  } while (0)
  if (y_dtype == MF_F32) PN_LAUNCH(float);
  if (y_dtype == MF_BF16) PN_LAUNCH(__nv_bfloat16);
#undef PN_LAUNCH
#undef PN_VEC
  return MF_ERR_BAD_DTYPE;
}
