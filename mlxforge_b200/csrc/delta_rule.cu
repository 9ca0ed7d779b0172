// Gated delta rule with one decay per head and key channel, and what stands around it.
//
// Per head, with a state S [dim, vdim] in 32-bit that is carried from token to token:
//   S <- diag(g_t) S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
// (the read-out sees the token's own write).  Queries and keys come from a short causal
// convolution over time per channel and SiLU, are made unit vectors per head
// (x / sqrt(sum x^2 + 1e-6)), the query also times dim^-1/2; values pass their own convolution
// and SiLU.  g_t = exp(-exp(A_log_h) softplus(a_t + dt_bias)), beta_t = sigmoid(b_t).  The
// read-out of a head is divided by its root mean square over vdim, multiplied by a weight and
// by a sigmoid gate.  Everything after the projections is 32-bit.
//
// Every column of S is independent of the others: u_c = beta (v_c - S[:, c] . k) touches
// column c only.  So the recurrence runs in parallel over (sequence, head, column) and is
// serial in time only; a column is shared by 8 lanes that hold dim/8 rows each in registers.
// The state after a token is the same however the prompt was cut: a step continues from the
// state in the request's slot.
//
// The slot also keeps the last taps-1 inputs of the convolutions, [(taps-1), C] after S.
#include "common.cuh"

#define DR_LANES 8          // lanes that share a column of S
#define DR_COLS 16          // columns per block
#define DR_THREADS (DR_LANES * DR_COLS)

__device__ __forceinline__ float dr_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float dr_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------ convolution, SiLU, unit norms, beta
// proj [T, ld]: q | k | v channels (C of them), then n_heads beta logits, then `n_low` low-rank
// activations that are only copied (rounded to the compute dtype) into `low` [T, n_low].
// qkv_out [T, C] 32-bit: queries (unit, scaled), keys (unit), values.  beta_out [T, n_heads].
template <typename TL>
__global__ void __launch_bounds__(1024)
delta_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ conv_w, int taps,
                     const float* __restrict__ state, long long state_stride, long long conv_off,
                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                     const int* __restrict__ seq_q_start, const int* __restrict__ slots, float* __restrict__ qkv_out,
                     float* __restrict__ beta_out, TL* __restrict__ low, int n_low, int n_heads, int n_kv, int dim,
                     int vdim) {
  extern __shared__ float y[];        // [C]
  const int t = blockIdx.x;
  const int C = 2 * n_kv * dim + n_heads * vdim;
  const int seq = seq_of_token[t];
  const int rel = t - seq_q_start[seq];           // index of the token within its portion
  const float* tail = state + (long long)slots[seq] * state_stride + conv_off;   // [(taps-1), C]
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < taps; j++) {
      const int back = taps - 1 - j;
      float x;
      if (rel - back >= 0) x = proj[(long long)(t - back) * ld + c];
      else x = tail[(long long)(rel - back + taps - 1) * C + c];
      a = fmaf(conv_w[(long long)c * taps + j], x, a);
    }
    y[c] = a * dr_sigmoid(a);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* o = qkv_out + (long long)t * C;
  // unit vectors: 2 * n_kv heads of `dim` channels, a warp each
  for (int hh = warp; hh < 2 * n_kv; hh += nwarps) {
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(y[hh * dim + d], y[hh * dim + d], ss);
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + 1e-6f);
    if (hh < n_kv) inv *= 1.0f / sqrtf((float)dim);
    for (int d = lane; d < dim; d += 32) o[hh * dim + d] = y[hh * dim + d] * inv;
  }
  for (int c = 2 * n_kv * dim + threadIdx.x; c < C; c += blockDim.x) o[c] = y[c];
  const float* p = proj + (long long)t * ld;
  for (int h = threadIdx.x; h < n_heads; h += blockDim.x) beta_out[(long long)t * n_heads + h] = dr_sigmoid(p[C + h]);
  for (int i = threadIdx.x; i < n_low; i += blockDim.x) low[(long long)t * n_low + i] = from_f32<TL>(p[C + n_heads + i]);
}

// After the step the slot keeps the last taps-1 inputs of every channel.
__global__ void delta_conv_tail_kernel(const float* __restrict__ proj, int ld, int C, int taps, float* __restrict__ state,
                                       long long state_stride, long long conv_off, const int* __restrict__ seq_q_start,
                                       const int* __restrict__ seq_q_len, const int* __restrict__ slots) {
  const int seq = blockIdx.x;
  const int start = seq_q_start[seq], n = seq_q_len[seq];
  float* tail = state + (long long)slots[seq] * state_stride + conv_off;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    for (int j = 0; j < taps - 1; j++) {          // ascending: a read is never behind a write
      const int src = n - (taps - 1) + j;
      tail[(long long)j * C + c] = src >= 0 ? proj[(long long)(start + src) * ld + c] : tail[(long long)(j + n) * C + c];
    }
  }
}

// ------------------------------------------------------------------ decays and output gates
// ag [T, n_heads * dim + n_gate]: the first part becomes exp(-exp(A_log_h) softplus(x + dt_bias)),
// the rest sigmoid(x), in place.
__global__ void delta_gates_kernel(float* __restrict__ ag, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias, int n_decay, int dim, int width, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int j = (int)(i % width);
  const float x = ag[i];
  if (j < n_decay) ag[i] = expf(-expf(a_log[j / dim]) * dr_softplus(x + dt_bias[j]));
  else ag[i] = dr_sigmoid(x);
}

// ------------------------------------------------------------------ the recurrence
template <int DPT>
__global__ void __launch_bounds__(DR_THREADS)
delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ ag,
                        int ag_ld, float* __restrict__ state, long long state_stride, const int* __restrict__ seq_q_start,
                        const int* __restrict__ seq_q_len, const int* __restrict__ slots, float* __restrict__ o_out,
                        int n_heads, int n_kv, int dim, int vdim) {
  const int seq = blockIdx.x, h = blockIdx.y;
  const int col = blockIdx.z * DR_COLS + threadIdx.x / DR_LANES;
  const int part = threadIdx.x % DR_LANES;
  const int kvh = h / (n_heads / n_kv);
  const int C = 2 * n_kv * dim + n_heads * vdim;
  const int start = seq_q_start[seq], n = seq_q_len[seq];
  const bool live = col < vdim;
  float* S = state + (long long)slots[seq] * state_stride + (long long)h * dim * vdim;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = part * DPT + i;
    s[i] = (live && d < dim) ? S[(long long)d * vdim + col] : 0.f;
  }
  float kd[DPT], qd[DPT], gd[DPT];
  float v = 0.f, b = 0.f;
  auto fetch = [&](int t) {
    const float* row = qkv + (long long)t * C;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      const int d = part * DPT + i;
      const bool in = d < dim;
      qd[i] = in ? row[kvh * dim + d] : 0.f;
      kd[i] = in ? row[n_kv * dim + kvh * dim + d] : 0.f;
      gd[i] = in ? ag[(long long)t * ag_ld + h * dim + d] : 0.f;
    }
    v = live ? row[2 * n_kv * dim + h * vdim + col] : 0.f;
    b = beta[(long long)t * n_heads + h];
  };
  if (n > 0) fetch(start);
  for (int t = start; t < start + n; t++) {
    float kc[DPT], qc[DPT], gc[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      kc[i] = kd[i];
      qc[i] = qd[i];
      gc[i] = gd[i];
    }
    const float vc = v, bc = b;
    if (t + 1 < start + n) fetch(t + 1);          // the next token's operands are on their way meanwhile
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      s[i] *= gc[i];
      dot = fmaf(s[i], kc[i], dot);
    }
#pragma unroll
    for (int off = 1; off < DR_LANES; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float u = bc * (vc - dot);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      s[i] = fmaf(kc[i], u, s[i]);
      o = fmaf(s[i], qc[i], o);
    }
#pragma unroll
    for (int off = 1; off < DR_LANES; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
    if (live && part == 0) o_out[(long long)t * n_heads * vdim + h * vdim + col] = o;
  }
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = part * DPT + i;
    if (live && d < dim) S[(long long)d * vdim + col] = s[i];
  }
}

// The same recurrence with the operands of the coming tokens brought into shared memory ahead of
// time: stages of DR_CHUNK tokens (q, k and g rows of the head, the block's 16 values, beta) are
// copied by cp.async into a ring of DR_STAGES, so the serial loop over the tokens reads shared
// memory only and a token no longer waits for a round trip to memory.  Channel d of a column
// belongs to lane ((d / 4) % 8) of its eight lanes, so that the eight lanes read 128 consecutive
// bytes of a row at once.  Needs dim, vdim and the row lengths to be multiples of 4 (16-byte copies).
#define DR_CHUNK 8
#define DR_STAGES 4

__device__ __forceinline__ void dr_cp16(void* smem, const void* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void dr_cp4(void* smem, const void* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(addr), "l"(gmem) : "memory");
}

template <int DPT>
__global__ void __launch_bounds__(DR_THREADS)
delta_recurrence_staged_kernel(const float* __restrict__ qkv, const float* __restrict__ beta,
                               const float* __restrict__ ag, int ag_ld, float* __restrict__ state,
                               long long state_stride, const int* __restrict__ seq_q_start,
                               const int* __restrict__ seq_q_len, const int* __restrict__ slots,
                               float* __restrict__ o_out, int n_heads, int n_kv, int dim, int vdim) {
  constexpr int DP = DPT * DR_LANES;                         // channels, padded
  constexpr int TOK = 3 * DP + DR_COLS + 4;                  // floats of one token in a stage: q, k, g, v, beta
  extern __shared__ __align__(16) float dr_sm[];             // [DR_STAGES][DR_CHUNK][TOK]
  const int seq = blockIdx.x, h = blockIdx.y;
  const int col0 = blockIdx.z * DR_COLS;
  const int ci = threadIdx.x / DR_LANES, part = threadIdx.x % DR_LANES;
  const int col = col0 + ci;
  const int kvh = h / (n_heads / n_kv);
  const int C = 2 * n_kv * dim + n_heads * vdim;
  const int start = seq_q_start[seq], n = seq_q_len[seq];
  const bool live = col < vdim;
  // the padding of q, k, g and v is never copied: zero once, where there is any
  if (dim < DP || col0 + DR_COLS > vdim) {
    for (int i = threadIdx.x; i < DR_STAGES * DR_CHUNK * TOK; i += DR_THREADS) dr_sm[i] = 0.f;
    __syncthreads();
  }
  float* S = state + (long long)slots[seq] * state_stride + (long long)h * dim * vdim;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = ((i >> 2) * DR_LANES + part) * 4 + (i & 3);
    s[i] = (live && d < dim) ? S[(long long)d * vdim + col] : 0.f;
  }
  const int d4 = dim / 4;
  const int n_chunks = (n + DR_CHUNK - 1) / DR_CHUNK;
  // what this thread copies of every stage, worked out once: up to NP 16-byte pieces of the q, k and
  // g rows (source pointer for the first stage, it moves on by a stage's tokens; place in the stage),
  // one piece of the values and one beta
  constexpr int NP = (DR_CHUNK * 3 * (DP / 4) + DR_THREADS - 1) / DR_THREADS;
  const float* src[NP];
  int dst[NP], ptok[NP], pstep[NP];
#pragma unroll
  for (int p = 0; p < NP; p++) {
    const int i = threadIdx.x + p * DR_THREADS;
    ptok[p] = DR_CHUNK;                                   // no piece
    src[p] = qkv;
    dst[p] = 0;
    pstep[p] = 0;
    if (i < DR_CHUNK * 3 * d4) {
      const int tok = i / (3 * d4), rem = i - tok * 3 * d4;
      const int which = rem / d4, c = (rem - which * d4) * 4;
      const long long t = start + tok;
      ptok[p] = tok;
      src[p] = which == 0 ? qkv + t * C + kvh * dim + c
             : which == 1 ? qkv + t * C + (n_kv + kvh) * dim + c
                          : ag + t * ag_ld + h * dim + c;
      pstep[p] = DR_CHUNK * (which == 2 ? ag_ld : C);
      dst[p] = tok * TOK + which * DP + c;
    }
  }
  const int vtok = threadIdx.x / (DR_COLS / 4), vc = (threadIdx.x % (DR_COLS / 4)) * 4;      // 32 threads: 8 tokens x 4 pieces
  const bool vcopy = threadIdx.x < DR_CHUNK * (DR_COLS / 4) && col0 + vc < vdim;
  const float* vsrc = qkv + (long long)(start + vtok) * C + 2 * n_kv * dim + h * vdim + col0 + vc;
  const bool bcopy = threadIdx.x >= 64 && threadIdx.x < 64 + DR_CHUNK;
  const int btok = threadIdx.x - 64;
  const float* bsrc = beta + (long long)(start + btok) * n_heads + h;
  auto issue = [&](int chunk) {
    if (chunk < n_chunks) {
      float* st = dr_sm + (size_t)(chunk % DR_STAGES) * DR_CHUNK * TOK;
      const int nt = min(DR_CHUNK, n - chunk * DR_CHUNK);
#pragma unroll
      for (int p = 0; p < NP; p++)
        if (ptok[p] < nt) dr_cp16(st + dst[p], src[p] + (long long)chunk * pstep[p]);
      if (vcopy && vtok < nt) dr_cp16(st + vtok * TOK + 3 * DP + vc, vsrc + (long long)chunk * DR_CHUNK * C);
      if (bcopy && btok < nt) dr_cp4(st + btok * TOK + 3 * DP + DR_COLS, bsrc + (long long)chunk * DR_CHUNK * n_heads);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
#pragma unroll
  for (int c = 0; c < DR_STAGES - 1; c++) issue(c);
  for (int chunk = 0; chunk < n_chunks; chunk++) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(DR_STAGES - 2) : "memory");
    __syncthreads();                         // the stage has landed for all, and the stage read before is free
    issue(chunk + DR_STAGES - 1);
    const float* st = dr_sm + (size_t)(chunk % DR_STAGES) * DR_CHUNK * TOK;
    const int nt = min(DR_CHUNK, n - chunk * DR_CHUNK);
    for (int tok = 0; tok < nt; tok++) {
      const float* row = st + tok * TOK;
      const float4* q4 = reinterpret_cast<const float4*>(row);
      const float4* k4 = reinterpret_cast<const float4*>(row + DP);
      const float4* g4 = reinterpret_cast<const float4*>(row + 2 * DP);
      const float v = row[3 * DP + ci], b = row[3 * DP + DR_COLS];
      // a partial sum per group of four channels: independent chains
      float4 kk[DPT / 4];
      float dp[DPT / 4];
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; i4++) {
        const float4 g = g4[i4 * DR_LANES + part];
        kk[i4] = k4[i4 * DR_LANES + part];
        s[4 * i4] *= g.x; s[4 * i4 + 1] *= g.y; s[4 * i4 + 2] *= g.z; s[4 * i4 + 3] *= g.w;
        dp[i4] = fmaf(s[4 * i4 + 3], kk[i4].w, fmaf(s[4 * i4 + 2], kk[i4].z, fmaf(s[4 * i4 + 1], kk[i4].y, s[4 * i4] * kk[i4].x)));
      }
      float dot = dp[0];
#pragma unroll
      for (int i4 = 1; i4 < DPT / 4; i4++) dot += dp[i4];
#pragma unroll
      for (int off = 1; off < DR_LANES; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
      const float u = b * (v - dot);
      float op[DPT / 4];
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; i4++) {
        const float4 q = q4[i4 * DR_LANES + part];
        s[4 * i4] = fmaf(kk[i4].x, u, s[4 * i4]);
        s[4 * i4 + 1] = fmaf(kk[i4].y, u, s[4 * i4 + 1]);
        s[4 * i4 + 2] = fmaf(kk[i4].z, u, s[4 * i4 + 2]);
        s[4 * i4 + 3] = fmaf(kk[i4].w, u, s[4 * i4 + 3]);
        op[i4] = fmaf(s[4 * i4 + 3], q.w, fmaf(s[4 * i4 + 2], q.z, fmaf(s[4 * i4 + 1], q.y, s[4 * i4] * q.x)));
      }
      float o = op[0];
#pragma unroll
      for (int i4 = 1; i4 < DPT / 4; i4++) o += op[i4];
#pragma unroll
      for (int off = 1; off < DR_LANES; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (live && part == 0)
        o_out[(long long)(start + chunk * DR_CHUNK + tok) * n_heads * vdim + h * vdim + col] = o;
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = ((i >> 2) * DR_LANES + part) * 4 + (i & 3);
    if (live && d < dim) S[(long long)d * vdim + col] = s[i];
  }
}

// ------------------------------------------------------------------ read-out norm and gate
// out[t, h, c] = o[t, h, c] / sqrt(mean_c o^2 + eps) * w[c] * gate[t, h, c]; a warp per (token, head).
// w_per_head: the weight is [n_heads * vdim] (a row of its own for every head) instead of [vdim].
template <typename TO>
__global__ void __launch_bounds__(256)
delta_output_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_ld,
                    const float* __restrict__ w, float eps, TO* __restrict__ out, int n_heads, int vdim, int total,
                    int w_per_head) {
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= total) return;
  const int lane = threadIdx.x & 31;
  const int t = item / n_heads, h = item - t * n_heads;
  const float* row = o + (long long)item * vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) ss = fmaf(row[c], row[c], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  const float* g = gate + (long long)t * gate_ld + h * vdim;
  const float* wh = w + (w_per_head ? h * vdim : 0);
  for (int c = lane; c < vdim; c += 32) out[(long long)item * vdim + c] = from_f32<TO>(row[c] * inv * wh[c] * g[c]);
}

// ------------------------------------------------------------------ entry points
MF_API int mf_delta_prepare(const float* proj, int ld, const float* conv_w, int taps, float* state,
                            long long state_stride, long long conv_off, const int* positions, const int* seq_of_token,
                            const int* seq_q_start, const int* seq_q_len, const int* slots, float* qkv_out,
                            float* beta_out, void* low, int low_dtype, int n_low, int T, int n_seqs, int n_heads,
                            int n_kv, int dim, int vdim, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || n_kv <= 0 || n_heads % n_kv) return MF_ERR_BAD_ARG;
  const int C = 2 * n_kv * dim + n_heads * vdim;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return MF_ERR_BAD_ARG;
  mf_count(MF_K_DELTA_PREPARE);
#define DP_LAUNCH(TL)                                                                                              \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<TL>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    delta_prepare_kernel<TL><<<T, T <= 64 ? 1024 : 256, smem, stream>>>(proj, ld, conv_w, taps, state, state_stride, conv_off,      \
                                                       positions, seq_of_token, seq_q_start, slots, qkv_out,       \
                                                       beta_out, (TL*)low, n_low, n_heads, n_kv, dim, vdim);       \
  } while (0)
  if (low_dtype == MF_F32) DP_LAUNCH(float);
  else if (low_dtype == MF_BF16) DP_LAUNCH(__nv_bfloat16);
  else return MF_ERR_BAD_DTYPE;
#undef DP_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (taps > 1) {
    delta_conv_tail_kernel<<<n_seqs, 256, 0, stream>>>(proj, ld, C, taps, state, state_stride, conv_off, seq_q_start,
                                                       seq_q_len, slots);
    e = cudaGetLastError();
  }
  return (int)e;
}

MF_API int mf_delta_gates(float* ag, const float* a_log, const float* dt_bias, int T, int n_heads, int dim, int n_gate,
                          cudaStream_t stream) {
  if (T <= 0) return 0;
  const int width = n_heads * dim + n_gate;
  const long long total = (long long)T * width;
  mf_count(MF_K_DELTA_GATES);
  delta_gates_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(ag, a_log, dt_bias, n_heads * dim, dim, width,
                                                                         total);
  return (int)cudaGetLastError();
}

MF_API int mf_delta_recurrence(const float* qkv, const float* beta, const float* ag, int ag_ld, float* state,
                               long long state_stride, const int* seq_q_start, const int* seq_q_len, const int* slots,
                               float* o_out, int n_seqs, int n_heads, int n_kv, int dim, int vdim, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (dim <= 0 || dim > 32 * DR_LANES || n_kv <= 0 || n_heads % n_kv || n_heads > 65535) return MF_ERR_BAD_ARG;
  dim3 grid(n_seqs, n_heads, (vdim + DR_COLS - 1) / DR_COLS);
  mf_count(MF_K_DELTA_RECURRENCE);
#define DR_LAUNCH(DPT)                                                                                             \
  delta_recurrence_kernel<DPT><<<grid, DR_THREADS, 0, stream>>>(qkv, beta, ag, ag_ld, state, state_stride,         \
                                                                seq_q_start, seq_q_len, slots, o_out, n_heads, n_kv, \
                                                                dim, vdim)
  const int per = (dim + DR_LANES - 1) / DR_LANES;
  const bool aligned = dim % 4 == 0 && vdim % 4 == 0 && ag_ld % 4 == 0 && ((uintptr_t)qkv & 15) == 0 &&
                       ((uintptr_t)ag & 15) == 0;
  if (aligned) {
    // the staged kernel: operands through a cp.async ring in shared memory
#define DS_LAUNCH(DPT)                                                                                             \
  do {                                                                                                             \
    const size_t smem = (size_t)DR_STAGES * DR_CHUNK * (3 * DPT * DR_LANES + DR_COLS + 4) * sizeof(float);         \
    static DeviceOnce once;                                                                                        \
    const int dev = mf_current_device();                                                                           \
    if (dev < 0) return MF_ERR_BAD_ARG;                                                                            \
    if (!once.done[dev]) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(delta_recurrence_staged_kernel<DPT>,                                    \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      if (e != cudaSuccess) return (int)e;                                                                         \
      once.done[dev] = true;                                                                                       \
    }                                                                                                              \
    delta_recurrence_staged_kernel<DPT><<<grid, DR_THREADS, smem, stream>>>(                                       \
        qkv, beta, ag, ag_ld, state, state_stride, seq_q_start, seq_q_len, slots, o_out, n_heads, n_kv, dim, vdim); \
  } while (0)
    if (per <= 4) DS_LAUNCH(4);
    else if (per <= 8) DS_LAUNCH(8);
    else if (per <= 16) DS_LAUNCH(16);
    else DS_LAUNCH(32);
#undef DS_LAUNCH
    return (int)cudaGetLastError();
  }
  if (per <= 4) DR_LAUNCH(4);
  else if (per <= 8) DR_LAUNCH(8);
  else if (per <= 16) DR_LAUNCH(16);
  else DR_LAUNCH(32);
#undef DR_LAUNCH
  return (int)cudaGetLastError();
}

MF_API int mf_delta_output(const float* o, const float* gate, int gate_ld, const float* w, float eps, void* out,
                           int out_dtype, int T, int n_heads, int vdim, int w_per_head, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int total = T * n_heads;
  const unsigned blocks = (unsigned)((total + 7) / 8);
  mf_count(MF_K_DELTA_OUTPUT);
  if (out_dtype == MF_F32)
    delta_output_kernel<float><<<blocks, 256, 0, stream>>>(o, gate, gate_ld, w, eps, (float*)out, n_heads, vdim, total,
                                                           w_per_head);
  else if (out_dtype == MF_BF16)
    delta_output_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(o, gate, gate_ld, w, eps, (__nv_bfloat16*)out,
                                                                   n_heads, vdim, total, w_per_head);
  else
    return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ decays and gates from rows of their own
// ag [T, n_heads * dim + n_gate] from two inputs.  Decays, one per head and key channel: the input has one
// number per head and channel, or (per_head) one per head that all its channels share;
//   kind 0: exp(-exp(a_log[h]) softplus(x + bias)) ,   kind 1: exp(-c sigmoid(x + bias))
// (bias indexed like the input).  Gates: sigmoid (gate_act 0) or SiLU (1) of gate_in.
__global__ void delta_gates_ex_kernel(const float* __restrict__ decay_in, int decay_ld, int per_head, int kind, float c,
                                      const float* __restrict__ a_log, const float* __restrict__ bias,
                                      const float* __restrict__ gate_in, int gate_ld, int gate_act,
                                      float* __restrict__ ag, int n_decay, int dim, int width, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / width;
  const int j = (int)(i - t * width);
  if (j < n_decay) {
    const int h = j / dim, src = per_head ? h : j;
    const float x = decay_in[t * decay_ld + src] + (bias ? bias[src] : 0.f);
    ag[i] = kind == 0 ? expf(-expf(a_log[h]) * dr_softplus(x)) : expf(-c * dr_sigmoid(x));
  } else {
    const float x = gate_in[t * gate_ld + (j - n_decay)];
    ag[i] = gate_act == 0 ? dr_sigmoid(x) : x * dr_sigmoid(x);
  }
}

MF_API int mf_delta_gates_ex(const float* decay_in, int decay_ld, int per_head, int kind, float c, const float* a_log,
                             const float* bias, const float* gate_in, int gate_ld, int gate_act, float* ag, int T,
                             int n_heads, int dim, int n_gate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (kind < 0 || kind > 1 || (kind == 0 && !a_log) || gate_act < 0 || gate_act > 1) return MF_ERR_BAD_ARG;
  const int width = n_heads * dim + n_gate;
  const long long total = (long long)T * width;
  mf_count(MF_K_DELTA_GATES);
  delta_gates_ex_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
      decay_in, decay_ld, per_head, kind, c, a_log, bias, gate_in, gate_ld, gate_act, ag, n_heads * dim, dim, width, total);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ generalized delta rule
// Per head, with a 32-bit state S [dim, dim]:
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T ,   o_t = S_t^T r_t
// with u = k / sqrt(sum k^2 + 1e-6) the unit key of the head; the decay and the removal both read the
// OLD state.  Column c of S needs only column c, so the recurrence is parallel over (sequence, head,
// column) and serial in time, as above.
//
// gdelta_prepare: proj [T, ld] 32-bit holds r | k | v | a | (gate) | low, each n = n_heads * dim wide but
// the last (`rank`).  ops_out [T, 4 n] gets r | k | u | a u with a = sigmoid(a + a_bias); `low` [T, rank]
// gets tanh of the low-rank activations in the compute dtype.
template <typename TL>
__global__ void __launch_bounds__(256)
gdelta_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ a_bias,
                      float* __restrict__ ops_out, TL* __restrict__ low, int low_off, int rank, int n_heads, int dim) {
  const long long t = blockIdx.x;
  const int n = n_heads * dim;
  const float* p = proj + t * ld;
  float* o = ops_out + t * 4 * n;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = warp; h < n_heads; h += nwarps) {
    const float* k = p + n + h * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(k[d], k[d], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + 1e-6f);
    for (int d = lane; d < dim; d += 32) {
      const int c = h * dim + d;
      const float u = k[d] * inv;
      o[c] = p[c];
      o[n + c] = k[d];
      o[2 * n + c] = u;
      o[3 * n + c] = dr_sigmoid(p[3 * n + c] + (a_bias ? a_bias[c] : 0.f)) * u;
    }
  }
  for (int i = threadIdx.x; i < rank; i += blockDim.x) low[t * rank + i] = from_f32<TL>(tanhf(p[low_off + i]));
}

MF_API int mf_gdelta_prepare(const float* proj, int ld, const float* a_bias, float* ops_out, void* low, int low_dtype,
                             int low_off, int rank, int T, int n_heads, int dim, cudaStream_t stream) {
  if (T <= 0) return 0;
  mf_count(MF_K_GDELTA_PREPARE);
  if (low_dtype == MF_F32)
    gdelta_prepare_kernel<float><<<T, 256, 0, stream>>>(proj, ld, a_bias, ops_out, (float*)low, low_off, rank, n_heads, dim);
  else if (low_dtype == MF_BF16)
    gdelta_prepare_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>(proj, ld, a_bias, ops_out, (__nv_bfloat16*)low, low_off,
                                                                rank, n_heads, dim);
  else
    return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}

// ops [T, 4 n]: r | k | u | a u;  w [T, w_ld]: the decays of head h at column h * dim;  v [T, v_ld]: the
// values of head h at column h * dim (32-bit).  Channel d of a column belongs to lane d / DPT of its eight.
template <int DPT>
__global__ void __launch_bounds__(DR_THREADS)
gdelta_recurrence_kernel(const float* __restrict__ ops, const float* __restrict__ w, int w_ld,
                         const float* __restrict__ v, int v_ld, float* __restrict__ state, long long state_stride,
                         const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                         const int* __restrict__ slots, float* __restrict__ o_out, int n_heads, int dim) {
  const int seq = blockIdx.x, h = blockIdx.y;
  const int col = blockIdx.z * DR_COLS + threadIdx.x / DR_LANES;
  const int part = threadIdx.x % DR_LANES;
  const int n = n_heads * dim;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const bool live = col < dim;
  float* S = state + (long long)slots[seq] * state_stride + (long long)h * dim * dim;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = part * DPT + i;
    s[i] = (live && d < dim) ? S[(long long)d * dim + col] : 0.f;
  }
  float rd[DPT], kd[DPT], ud[DPT], ad[DPT], wd[DPT];
  float vv = 0.f;
  auto fetch = [&](int t) {
    const float* row = ops + (long long)t * 4 * n + h * dim;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      const int d = part * DPT + i;
      const bool in = d < dim;
      rd[i] = in ? row[d] : 0.f;
      kd[i] = in ? row[n + d] : 0.f;
      ud[i] = in ? row[2 * n + d] : 0.f;
      ad[i] = in ? row[3 * n + d] : 0.f;
      wd[i] = in ? w[(long long)t * w_ld + h * dim + d] : 0.f;
    }
    vv = live ? v[(long long)t * v_ld + h * dim + col] : 0.f;
  };
  if (len > 0) fetch(start);
  for (int t = start; t < start + len; t++) {
    float rc[DPT], kc[DPT], uc[DPT], ac[DPT], wc[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      rc[i] = rd[i];
      kc[i] = kd[i];
      uc[i] = ud[i];
      ac[i] = ad[i];
      wc[i] = wd[i];
    }
    const float vc = vv;
    if (t + 1 < start + len) fetch(t + 1);        // the next token's operands are on their way meanwhile
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; i++) dot = fmaf(s[i], uc[i], dot);
#pragma unroll
    for (int off = 1; off < DR_LANES; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      s[i] = fmaf(kc[i], vc, fmaf(-ac[i], dot, wc[i] * s[i]));
      o = fmaf(s[i], rc[i], o);
    }
#pragma unroll
    for (int off = 1; off < DR_LANES; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
    if (live && part == 0) o_out[(long long)t * n + h * dim + col] = o;
  }
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = part * DPT + i;
    if (live && d < dim) S[(long long)d * dim + col] = s[i];
  }
}

// The same with the operands of the coming tokens brought into shared memory ahead of time, as the gated
// rule's staged kernel does: stages of DR_CHUNK tokens (the r, k, u, a u and w rows of the head and the
// block's values) arrive by cp.async in a ring of DR_STAGES; LANES lanes share a column and COLS columns a
// block; channel d of a column belongs to lane ((d / 4) % LANES).  A token's chain of instructions in a warp
// is what bounds the kernel, so heads of more than 32 channels are spread over 16 lanes (fewer instructions a
// lane and token) in blocks of 8 columns (less of the operands read again by every column).  Needs dim and
// the row lengths to be multiples of 4 (16-byte copies).
template <int DPT, int LANES, int COLS>
__global__ void __launch_bounds__(LANES * COLS)
gdelta_recurrence_staged_kernel(const float* __restrict__ ops, const float* __restrict__ w, int w_ld,
                                const float* __restrict__ v, int v_ld, float* __restrict__ state,
                                long long state_stride, const int* __restrict__ seq_q_start,
                                const int* __restrict__ seq_q_len, const int* __restrict__ slots,
                                float* __restrict__ o_out, int n_heads, int dim) {
  constexpr int THREADS = LANES * COLS;
  constexpr int DP = DPT * LANES;                         // channels, padded
  constexpr int TOK = 5 * DP + COLS;                      // floats of one token in a stage: r, k, u, au, w, v
  extern __shared__ __align__(16) float gd_sm[];             // [DR_STAGES][DR_CHUNK][TOK]
  const int seq = blockIdx.x, h = blockIdx.y;
  const int col0 = blockIdx.z * COLS;
  const int ci = threadIdx.x / LANES, part = threadIdx.x % LANES;
  const int col = col0 + ci;
  const int n = n_heads * dim;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const bool live = col < dim;
  if (dim < DP || col0 + COLS > dim) {                    // the padding is never copied: zero once
    for (int i = threadIdx.x; i < DR_STAGES * DR_CHUNK * TOK; i += THREADS) gd_sm[i] = 0.f;
    __syncthreads();
  }
  float* S = state + (long long)slots[seq] * state_stride + (long long)h * dim * dim;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = ((i >> 2) * LANES + part) * 4 + (i & 3);
    s[i] = (live && d < dim) ? S[(long long)d * dim + col] : 0.f;
  }
  const int d4 = dim / 4;
  const int n_chunks = (len + DR_CHUNK - 1) / DR_CHUNK;
  // what this thread copies of every stage, worked out once: 16-byte pieces of the five rows, one of the values
  constexpr int NP = (DR_CHUNK * 5 * (DP / 4) + THREADS - 1) / THREADS;
  const float* src[NP];
  int dst[NP], ptok[NP], pstep[NP];
#pragma unroll
  for (int p = 0; p < NP; p++) {
    const int i = threadIdx.x + p * THREADS;
    ptok[p] = DR_CHUNK;                                   // no piece
    src[p] = ops;
    dst[p] = 0;
    pstep[p] = 0;
    if (i < DR_CHUNK * 5 * d4) {
      const int tok = i / (5 * d4), rem = i - tok * 5 * d4;
      const int which = rem / d4, c = (rem - which * d4) * 4;
      const long long t = start + tok;
      ptok[p] = tok;
      src[p] = which < 4 ? ops + t * 4 * n + (long long)which * n + h * dim + c : w + t * w_ld + h * dim + c;
      pstep[p] = DR_CHUNK * (which < 4 ? 4 * n : w_ld);
      dst[p] = tok * TOK + which * DP + c;
    }
  }
  const int vtok = threadIdx.x / (COLS / 4), vc = (threadIdx.x % (COLS / 4)) * 4;      // 32 threads: 8 tokens x 4 pieces
  const bool vcopy = threadIdx.x < DR_CHUNK * (COLS / 4) && col0 + vc < dim;
  const float* vsrc = v + (long long)(start + vtok) * v_ld + h * dim + col0 + vc;
  auto issue = [&](int chunk) {
    if (chunk < n_chunks) {
      float* st = gd_sm + (size_t)(chunk % DR_STAGES) * DR_CHUNK * TOK;
      const int nt = min(DR_CHUNK, len - chunk * DR_CHUNK);
#pragma unroll
      for (int p = 0; p < NP; p++)
        if (ptok[p] < nt) dr_cp16(st + dst[p], src[p] + (long long)chunk * pstep[p]);
      if (vcopy && vtok < nt) dr_cp16(st + vtok * TOK + 5 * DP + vc, vsrc + (long long)chunk * DR_CHUNK * v_ld);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
#pragma unroll
  for (int c = 0; c < DR_STAGES - 1; c++) issue(c);
  for (int chunk = 0; chunk < n_chunks; chunk++) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(DR_STAGES - 2) : "memory");
    __syncthreads();                         // the stage has landed for all, and the stage read before is free
    issue(chunk + DR_STAGES - 1);
    const float* st = gd_sm + (size_t)(chunk % DR_STAGES) * DR_CHUNK * TOK;
    const int nt = min(DR_CHUNK, len - chunk * DR_CHUNK);
    for (int tok = 0; tok < nt; tok++) {
      const float* row = st + tok * TOK;
      const float4* r4 = reinterpret_cast<const float4*>(row);
      const float4* k4 = reinterpret_cast<const float4*>(row + DP);
      const float4* u4 = reinterpret_cast<const float4*>(row + 2 * DP);
      const float4* a4 = reinterpret_cast<const float4*>(row + 3 * DP);
      const float4* w4 = reinterpret_cast<const float4*>(row + 4 * DP);
      const float vc_ = row[5 * DP + ci];
      float dp[DPT / 4];
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; i4++) {
        const float4 u = u4[i4 * LANES + part];
        dp[i4] = fmaf(s[4 * i4 + 3], u.w, fmaf(s[4 * i4 + 2], u.z, fmaf(s[4 * i4 + 1], u.y, s[4 * i4] * u.x)));
      }
      float dot = dp[0];
#pragma unroll
      for (int i4 = 1; i4 < DPT / 4; i4++) dot += dp[i4];
#pragma unroll
      for (int off = 1; off < LANES; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
      float op[DPT / 4];
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; i4++) {
        const float4 kk = k4[i4 * LANES + part], au = a4[i4 * LANES + part], ww = w4[i4 * LANES + part];
        const float4 r = r4[i4 * LANES + part];
        s[4 * i4] = fmaf(kk.x, vc_, fmaf(-au.x, dot, ww.x * s[4 * i4]));
        s[4 * i4 + 1] = fmaf(kk.y, vc_, fmaf(-au.y, dot, ww.y * s[4 * i4 + 1]));
        s[4 * i4 + 2] = fmaf(kk.z, vc_, fmaf(-au.z, dot, ww.z * s[4 * i4 + 2]));
        s[4 * i4 + 3] = fmaf(kk.w, vc_, fmaf(-au.w, dot, ww.w * s[4 * i4 + 3]));
        op[i4] = fmaf(s[4 * i4 + 3], r.w, fmaf(s[4 * i4 + 2], r.z, fmaf(s[4 * i4 + 1], r.y, s[4 * i4] * r.x)));
      }
      float o = op[0];
#pragma unroll
      for (int i4 = 1; i4 < DPT / 4; i4++) o += op[i4];
#pragma unroll
      for (int off = 1; off < LANES; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (live && part == 0) o_out[(long long)(start + chunk * DR_CHUNK + tok) * n + h * dim + col] = o;
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int d = ((i >> 2) * LANES + part) * 4 + (i & 3);
    if (live && d < dim) S[(long long)d * dim + col] = s[i];
  }
}

MF_API int mf_gdelta_recurrence(const float* ops, const float* w, int w_ld, const float* v, int v_ld, float* state,
                                long long state_stride, const int* seq_q_start, const int* seq_q_len, const int* slots,
                                float* o_out, int n_seqs, int n_heads, int dim, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (dim <= 0 || dim > 16 * DR_LANES || n_heads <= 0 || n_heads > 65535) return MF_ERR_BAD_ARG;
  mf_count(MF_K_GDELTA_RECURRENCE);
  const int per = (dim + DR_LANES - 1) / DR_LANES;
  const bool aligned = dim % 4 == 0 && w_ld % 4 == 0 && v_ld % 4 == 0 && ((uintptr_t)ops & 15) == 0 &&
                       ((uintptr_t)w & 15) == 0 && ((uintptr_t)v & 15) == 0;
  if (aligned) {
#define GS_LAUNCH(DPT, LANES, COLS)                                                                                \
  do {                                                                                                             \
    const size_t smem = (size_t)DR_STAGES * DR_CHUNK * (5 * DPT * LANES + COLS) * sizeof(float);                   \
    static DeviceOnce once;                                                                                        \
    const int dev = mf_current_device();                                                                           \
    if (dev < 0) return MF_ERR_BAD_ARG;                                                                            \
    if (!once.done[dev]) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(gdelta_recurrence_staged_kernel<DPT, LANES, COLS>,                      \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      if (e != cudaSuccess) return (int)e;                                                                         \
      once.done[dev] = true;                                                                                       \
    }                                                                                                              \
    const dim3 sgrid(n_seqs, n_heads, (dim + COLS - 1) / COLS);                                                    \
    gdelta_recurrence_staged_kernel<DPT, LANES, COLS><<<sgrid, LANES * COLS, smem, stream>>>(                      \
        ops, w, w_ld, v, v_ld, state, state_stride, seq_q_start, seq_q_len, slots, o_out, n_heads, dim);           \
  } while (0)
    if (dim <= 32) GS_LAUNCH(4, 8, 16);
    else if (dim <= 64) GS_LAUNCH(4, 16, 8);
    else GS_LAUNCH(8, 16, 8);
#undef GS_LAUNCH
    return (int)cudaGetLastError();
  }
  dim3 grid(n_seqs, n_heads, (dim + DR_COLS - 1) / DR_COLS);
#define GD_LAUNCH(DPT)                                                                                            \
  gdelta_recurrence_kernel<DPT><<<grid, DR_THREADS, 0, stream>>>(ops, w, w_ld, v, v_ld, state, state_stride,      \
                                                                 seq_q_start, seq_q_len, slots, o_out, n_heads, dim)
  if (per <= 4) GD_LAUNCH(4);
  else if (per <= 8) GD_LAUNCH(8);
  else GD_LAUNCH(16);
#undef GD_LAUNCH
  return (int)cudaGetLastError();
}
