// Mixture of experts: the router's choice and the experts' feed-forward.
//
// Router (32-bit): s = sigmoid(z) over E experts, or s = softmax(z) over them (`mode`).  The
// experts form `n_groups` equal groups of neighbours; a group's score is the sum of its two
// largest s, and only experts of the `keep` best groups can be chosen (n_groups = 0: no such
// limit).  The `top` allowed experts with the largest s + bias (`bias`: one number per expert
// that only steers the choice; none: s itself) are chosen; their weights are s * route_scale,
// without the bias and not renormalised.  Ties go to the lower index.
//
// Expert:  g = min(Wg x, limit),  u = clamp(Wu x, -limit, limit),
//          y = Wd ( g * sigmoid(alpha g) * (u + up_off) )
// with the weights of all experts stacked: w_gu [E, 2, ff, H] (gate rows, then up rows) and
// w_down [E, H, ff].  (limit = infinity, alpha = 1, up_off = 0: the plain SiLU-gated expert.)
//
// Identity experts: router outputs from `n_real` on have no matrices; such an expert returns its
// input.  The experts' kernels skip them and the weighted sum adds weight * x for them.  The sum
// can also add a shared branch that every token takes: sigmoid(gate logit of the token) * shared.
//
// mf_moe_rows is the kernel for few tokens and for the 32-bit path: a block per (token, chosen
// expert, slice of the expert's columns) streams its part of that expert's matrices once; the
// chosen experts' outputs are then added in the order of the choice, so a token's result does
// not depend on what else is in the batch.
#include "common.cuh"

__device__ __forceinline__ float moe_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------ router
// one warp per token; dynamic shared memory per warp: s[E], sel[E], gs[n_groups]
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int ldz, int E, int n_groups, int keep, int top, float route_scale,
                 int mode, const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights, int T) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  const int per_warp = 2 * E + (n_groups > 0 ? n_groups : 1);
  float* s = sm + warp * per_warp;
  float* sel = s + E;
  float* gs = sel + E;
  const float* zr = z + (long long)t * ldz;
  const bool renorm = (mode & 2) != 0;       // the chosen weights divided by their sum (+ 1e-20)
  if (mode & 1) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      s[e] = expf(zr[e] - m);
      sum += s[e];
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
  } else {
    for (int e = lane; e < E; e += 32) s[e] = moe_sigmoid(zr[e]);
  }
  for (int e = lane; e < E; e += 32) sel[e] = bias ? s[e] + bias[e] : s[e];
  __syncwarp();
  if (n_groups > 0) {
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float t1 = -INFINITY, t2 = -INFINITY;
      for (int i = 0; i < per; i++) {
        const float v = s[g * per + i];
        if (v > t1) { t2 = t1; t1 = v; }
        else if (v > t2) t2 = v;
      }
      gs[g] = t1 + (t2 == -INFINITY ? 0.f : t2);
    }
    __syncwarp();
    // the `keep` best groups stay; the others' experts cannot be chosen
    for (int round = 0; round < n_groups - keep; round++) {
      float worst = INFINITY;
      int wi = -1;
      for (int g = lane; g < n_groups; g += 32) {      // the worst group, ties to the higher index
        const float v = gs[g];
        if (v <= worst && v != INFINITY) { worst = v; wi = g; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, worst, o);
        const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
        if (oi >= 0 && (wi < 0 || ov < worst || (ov == worst && oi > wi))) { worst = ov; wi = oi; }
      }
      if (wi >= 0) {
        for (int i = lane; i < per; i += 32) sel[wi * per + i] = -INFINITY;
        if (lane == 0) gs[wi] = INFINITY;              // out of the running
      }
      __syncwarp();
    }
  }
  float chosen_sum = 0.f;
  for (int k = 0; k < top; k++) {
    float best = -INFINITY;
    int bi = -1;
    for (int e = lane; e < E; e += 32) {
      const float v = sel[e];
      if (v > best) { best = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      ids[(long long)t * top + k] = bi < 0 ? 0 : bi;
      weights[(long long)t * top + k] = bi < 0 ? 0.f : s[bi] * route_scale;
      if (bi >= 0) {
        chosen_sum += s[bi];
        sel[bi] = -INFINITY;
      }
    }
    __syncwarp();
  }
  if (renorm && lane == 0) {
    const float inv = 1.0f / (chosen_sum + 1e-20f);
    for (int k = 0; k < top; k++) weights[(long long)t * top + k] *= inv;
  }
}

MF_API int mf_moe_route(const float* z, int ldz, int T, int E, int n_groups, int keep, int top, float route_scale,
                        int mode, const float* bias, int* ids, float* weights, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || ldz < E || mode < 0 || mode > 3) return MF_ERR_BAD_ARG;
  if (n_groups > 0 && (E % n_groups || keep < 1 || keep > n_groups || (long long)keep * (E / n_groups) < top))
    return MF_ERR_BAD_ARG;
  const int per_warp = 2 * E + (n_groups > 0 ? n_groups : 1);
  const size_t smem = (size_t)4 * per_warp * sizeof(float);
  if (smem > 48 * 1024) return MF_ERR_BAD_ARG;
  mf_count(MF_K_MOE_ROUTE);
  moe_route_kernel<<<(T + 3) / 4, 128, smem, stream>>>(z, ldz, E, n_groups, keep, top, route_scale, mode, bias, ids,
                                                       weights, T);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ experts, a block per (token, choice, slice)
// The expert's ff columns are cut into slices of MOE_SLICE: a block computes the activations of
// its slice and their share of the down projection, y [T, top, n_slices, H] 32-bit, not yet
// weighted.  The slices are fixed by ff alone, so a token's sums never depend on the batch.
#define MOE_SLICE 64

template <typename T>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const T* __restrict__ x, const T* __restrict__ w_gu, const T* __restrict__ w_down,
                const int* __restrict__ ids, float* __restrict__ y, int H, int ff, int top, float limit, float alpha,
                float up_off, int n_real, int act_kind) {
  extern __shared__ float sm[];
  float* xs = sm;            // [H]
  float* act = sm + H;       // [MOE_SLICE]
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, k = blockIdx.y, slice = blockIdx.z;
  const int f0 = slice * MOE_SLICE, fn = min(MOE_SLICE, ff - f0);
  const int e = ids[(long long)t * top + k];
  if (e >= n_real) return;     // an identity expert: the weighted sum takes the input itself
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < H; i += blockDim.x) xs[i] = to_f32<T>(x[(long long)t * H + i]);
  __syncthreads();
  // act_kind >= 0: an expert without a gate, down(act(up x)); its first matrix is [ff, H] alone
  const bool gated = act_kind < 0;
  const T* wg = w_gu + (long long)e * (gated ? 2 : 1) * ff * H;
  const T* wu = wg + (long long)ff * H;
  for (int f = warp; f < fn; f += nwarps) {
    const T* rg = wg + (long long)(f0 + f) * H;
    const T* ru = wu + (long long)(f0 + f) * H;
    float g = 0.f, u = 0.f;
    for (int i = lane; i < H; i += 32) {
      g = fmaf(xs[i], to_f32<T>(rg[i]), g);
      if (gated) u = fmaf(xs[i], to_f32<T>(ru[i]), u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0 && !gated) act[f] = to_f32<T>(from_f32<T>(gate_act(g, act_kind)));
    else if (lane == 0) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      // the activation is rounded where a product in the compute dtype would read it
      act[f] = to_f32<T>(from_f32<T>(g * moe_sigmoid(alpha * g) * (u + up_off)));
    }
  }
  __syncthreads();
  const T* wd = w_down + (long long)e * H * ff + f0;
  float* yo = y + (((long long)t * top + k) * gridDim.z + slice) * H;
  for (int c = warp; c < H; c += nwarps) {
    const T* rd = wd + (long long)c * ff;
    float a = 0.f;
    for (int i = lane; i < fn; i += 32) a = fmaf(act[i], to_f32<T>(rd[i]), a);
    a = warp_sum(a);
    if (lane == 0) yo[c] = a;
  }
}

// The same for bfloat16 in 16-byte pieces (H and ff multiples of 8): a warp per gate/up row with
// 8 columns a lane and pass, 8 lanes per row of the down projection's slice.
__device__ __forceinline__ float moe_dot8(const uint4 w, const float* xv) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&w);
  float a = 0.f;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const float2 f = __bfloat1622float2(p[j]);
    a = fmaf(xv[2 * j], f.x, a);
    a = fmaf(xv[2 * j + 1], f.y, a);
  }
  return a;
}

__global__ void __launch_bounds__(256)
moe_rows_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_gu,
                         const __nv_bfloat16* __restrict__ w_down, const int* __restrict__ ids, float* __restrict__ y,
                         int H, int ff, int top, float limit, float alpha, float up_off, int n_real, int act_kind) {
  extern __shared__ __align__(16) float sm[];
  float* xs = sm;            // [H]
  float* act = sm + H;       // [MOE_SLICE]
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, k = blockIdx.y, slice = blockIdx.z;
  const int f0 = slice * MOE_SLICE, fn = min(MOE_SLICE, ff - f0);
  const int e = ids[(long long)t * top + k];
  if (e >= n_real) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < H; i += blockDim.x) xs[i] = __bfloat162float(x[(long long)t * H + i]);
  if (threadIdx.x < MOE_SLICE) act[threadIdx.x] = 0.f;
  __syncthreads();
  const bool gated = act_kind < 0;
  const __nv_bfloat16* wg = w_gu + (long long)e * (gated ? 2 : 1) * ff * H;
  const __nv_bfloat16* wu = wg + (long long)ff * H;
  for (int f = warp; f < fn; f += nwarps) {
    const uint4* rg = reinterpret_cast<const uint4*>(wg + (long long)(f0 + f) * H);
    const uint4* ru = reinterpret_cast<const uint4*>(wu + (long long)(f0 + f) * H);
    float g = 0.f, u = 0.f;
    for (int i = lane; i < H / 8; i += 32) {
      const uint4 a = rg[i];
      float xv[8];
      *reinterpret_cast<float4*>(xv) = *reinterpret_cast<const float4*>(xs + 8 * i);
      *reinterpret_cast<float4*>(xv + 4) = *reinterpret_cast<const float4*>(xs + 8 * i + 4);
      g += moe_dot8(a, xv);
      if (gated) u += moe_dot8(ru[i], xv);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0 && !gated) act[f] = __bfloat162float(__float2bfloat16_rn(gate_act(g, act_kind)));
    else if (lane == 0) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      act[f] = __bfloat162float(__float2bfloat16_rn(g * moe_sigmoid(alpha * g) * (u + up_off)));
    }
  }
  __syncthreads();
  const __nv_bfloat16* wd = w_down + (long long)e * H * ff + f0;
  float* yo = y + (((long long)t * top + k) * gridDim.z + slice) * H;
  const int sub = threadIdx.x & 7, row0 = threadIdx.x >> 3;        // 8 lanes a row, 32 rows a pass
  float av[8];
  *reinterpret_cast<float4*>(av) = *reinterpret_cast<const float4*>(act + 8 * sub);
  *reinterpret_cast<float4*>(av + 4) = *reinterpret_cast<const float4*>(act + 8 * sub + 4);
  for (int c = row0; c < H; c += 32) {
    float a = 0.f;
    if (8 * sub < fn) a = moe_dot8(*reinterpret_cast<const uint4*>(wd + (long long)c * ff + 8 * sub), av);
    a += __shfl_xor_sync(0xffffffffu, a, 1);
    a += __shfl_xor_sync(0xffffffffu, a, 2);
    a += __shfl_xor_sync(0xffffffffu, a, 4);
    if (sub == 0) yo[c] = a;
  }
}

MF_API int mf_moe_rows_slices(int ff) { return (ff + MOE_SLICE - 1) / MOE_SLICE; }

MF_API int mf_moe_rows(const void* x, const void* w_gu, const void* w_down, int dtype, const int* ids, float* y, int T,
                       int H, int ff, int top, float limit, float alpha, float up_off, int n_real, int act_kind,
                       cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)(H + MOE_SLICE) * sizeof(float);
  if (smem > 200 * 1024 || top > 65535 || act_kind >= MF_ACT_COUNT) return MF_ERR_BAD_ARG;
  const dim3 grid(T, top, mf_moe_rows_slices(ff));
  mf_count(MF_K_MOE_ROWS);
#define MR_LAUNCH(KERNEL, TT)                                                                                      \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    return (int)launch_dep(KERNEL, grid, dim3(256), smem, stream, (const TT*)x, (const TT*)w_gu, (const TT*)w_down, \
                           ids, y, H, ff, top, limit, alpha, up_off, n_real, act_kind);                            \
  } while (0)
  if (dtype == MF_F32) MR_LAUNCH(moe_rows_kernel<float>, float);
  if (dtype == MF_BF16) {
    const bool vec = H % 8 == 0 && ff % 8 == 0 && ((uintptr_t)w_gu & 15) == 0 && ((uintptr_t)w_down & 15) == 0;
    if (vec) MR_LAUNCH(moe_rows_bf16_vec_kernel, __nv_bfloat16);
    MR_LAUNCH(moe_rows_kernel<__nv_bfloat16>, __nv_bfloat16);
  }
#undef MR_LAUNCH
  return MF_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ the weighted sum of the chosen experts
// out[t] = sum_k weights[t, k] * sum_s y[src(t, k) * slices + s], k in the order of the choice,
// the slices of an expert in their order.  `slot_of` null: src(t, k) = t * top + k; else the row
// of y that holds the pair (tokens sorted by expert).  With `ids` and `x`: a chosen expert from
// `n_real` on is an identity expert, whose output is x[t].  With `shared`: the token's row of it,
// times sigmoid(shared_gate[t * gate_ld]) where a gate is given, is added last.
struct MoeExtras {
  const int* ids;
  int n_real;
  const void* x;
  const void* shared;
  const float* shared_gate;
  int gate_ld;
};

template <typename TO, typename TY>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const TY* __restrict__ y, const float* __restrict__ weights, const int* __restrict__ slot_of,
                   TO* __restrict__ out, int H, int top, int slices, MoeExtras ex) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const TO* x = reinterpret_cast<const TO*>(ex.x);
  const TO* shared = reinterpret_cast<const TO*>(ex.shared);
  const float sg = shared ? (ex.shared_gate ? moe_sigmoid(ex.shared_gate[(long long)t * ex.gate_ld]) : 1.0f) : 0.f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; k++) {
      float part = 0.f;
      if (ex.ids && ex.ids[(long long)t * top + k] >= ex.n_real) {
        part = to_f32<TO>(x[(long long)t * H + i]);
      } else {
        const long long row = (slot_of ? slot_of[(long long)t * top + k] : (long long)t * top + k) * slices;
        for (int sl = 0; sl < slices; sl++) part += to_f32<TY>(y[(row + sl) * H + i]);
      }
      a = fmaf(weights[(long long)t * top + k], part, a);
    }
    if (shared) a = fmaf(sg, to_f32<TO>(shared[(long long)t * H + i]), a);
    out[(long long)t * H + i] = from_f32<TO>(a);
  }
}

// bfloat16 rows in 16-byte pieces (H a multiple of 8, one partial sum per pair): 8 columns a thread;
// identity experts and the shared branch as in the kernel above
__global__ void __launch_bounds__(256)
moe_combine_bf16_vec_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ weights,
                            const int* __restrict__ slot_of, __nv_bfloat16* __restrict__ out, int H, int top,
                            MoeExtras ex) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= H) return;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(ex.x);
  const __nv_bfloat16* shared = reinterpret_cast<const __nv_bfloat16*>(ex.shared);
  float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < top; k++) {
    const float wk = weights[(long long)t * top + k];
    const __nv_bfloat16* src;
    if (ex.ids && ex.ids[(long long)t * top + k] >= ex.n_real) {
      src = x + (long long)t * H + i;              // an identity expert returns the token's input
    } else {
      const long long row = slot_of ? slot_of[(long long)t * top + k] : (long long)t * top + k;
      src = y + row * H + i;
    }
    const uint4 v = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 f = __bfloat1622float2(p[j]);
      a[2 * j] = fmaf(wk, f.x, a[2 * j]);
      a[2 * j + 1] = fmaf(wk, f.y, a[2 * j + 1]);
    }
  }
  if (shared) {
    const float sg = ex.shared_gate ? moe_sigmoid(ex.shared_gate[(long long)t * ex.gate_ld]) : 1.0f;
    const uint4 v = *reinterpret_cast<const uint4*>(shared + (long long)t * H + i);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 f = __bfloat1622float2(p[j]);
      a[2 * j] = fmaf(sg, f.x, a[2 * j]);
      a[2 * j + 1] = fmaf(sg, f.y, a[2 * j + 1]);
    }
  }
  uint4 o;
  __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; j++) q[j] = __floats2bfloat162_rn(a[2 * j], a[2 * j + 1]);
  *reinterpret_cast<uint4*>(out + (long long)t * H + i) = o;
}

MF_API int mf_moe_combine(const void* y, int y_dtype, const float* weights, const int* slot_of, void* out, int out_dtype,
                          int T, int H, int top, int slices, const int* ids, int n_real, const void* x,
                          const void* shared, const float* shared_gate, int gate_ld, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (ids && !x) return MF_ERR_BAD_ARG;
  const MoeExtras ex{ids, n_real, x, shared, shared_gate, gate_ld};
  mf_count(MF_K_MOE_COMBINE);
  if (y_dtype == MF_BF16 && out_dtype == MF_BF16 && slices == 1 && H % 8 == 0 &&
      (((uintptr_t)y | (uintptr_t)out | (uintptr_t)x | (uintptr_t)shared) & 15) == 0)
    return (int)launch_dep(moe_combine_bf16_vec_kernel, dim3(T, (H / 8 + 255) / 256), dim3(256), 0, stream,
                           (const __nv_bfloat16*)y, weights, slot_of, (__nv_bfloat16*)out, H, top, ex);
  const dim3 grid(T, (H + 255) / 256);
#define MC_LAUNCH(TO, TY)                                                                                       \
  return (int)launch_dep(moe_combine_kernel<TO, TY>, grid, dim3(256), 0, stream, (const TY*)y, weights, slot_of, \
                         (TO*)out, H, top, slices, ex)
  if (y_dtype == MF_F32 && out_dtype == MF_F32) MC_LAUNCH(float, float);
  if (y_dtype == MF_F32 && out_dtype == MF_BF16) MC_LAUNCH(__nv_bfloat16, float);
  if (y_dtype == MF_BF16 && out_dtype == MF_BF16) MC_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef MC_LAUNCH
  return MF_ERR_BAD_DTYPE;
}
