// Experts for many tokens: the (token, choice) pairs are ordered by expert and every expert's
// pairs go through tensor-core tiles, so an expert's matrices are read once per tile of 64 pairs
// instead of once per pair.  The formulas are those of moe.cu.
//
//   mf_moe_sort     one block: counts per expert, offsets, a row for every pair (slot_of), the
//                   token of every row (row_token), and the list of tiles (expert, first row, rows).
//                   Pairs whose expert is `n_real` or above (identity experts, which have no
//                   matrices) get no row: slot_of is -1 for them.
//                   Which row a pair gets inside its expert's range is not fixed, and need not be:
//                   every row is computed by itself, and the sum over a token's experts is taken in
//                   the order of the choice by the combine kernel.
//                   `ends` [E] (optional): the row at which every expert's range ends.
//   mf_moe_gather_rows, mf_moe_activation   for the path through the library's grouped product
//                   (the engine uses library products for its other many-row projections too): the
//                   tokens' rows copied into the order of the rows, and the clamped activation of a
//                   [rows, 2 ff] product (gate columns, then up columns).
//   mf_moe_grouped_up    act[row] = g sigmoid(alpha g) (u + 1) with g, u the clamped gate and up
//                   products of the row's token (gathered by row_token), bfloat16.
//   mf_moe_grouped_down  y[row] = Wd_e act[row], 32-bit.
//
// Both products are mma.sync m16n8k16 tiles of 64 rows x 64 columns, four warps, K in steps of 64
// through two cp.async stages of shared memory: the next step's operands are on their way while
// this step's are multiplied.  The launches cover the largest possible number of tiles (known on the
// host: pairs / 64 + experts); blocks beyond the count the sort kernel wrote return at once, so a
// step's launches do not depend on its data.
#include "common.cuh"

#define MG_BM 64
#define MG_BN 64
#define MG_BK 64
#define MG_LD (MG_BK + 8)
#define MG_STAGES 2
#define MG_MAX_EXPERTS 1024

__device__ __forceinline__ void mg_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// meta: [0] number of tiles; tiles: [max_tiles][3] = expert, first row, rows
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int E, int top, int* __restrict__ slot_of,
                int* __restrict__ row_token, int* __restrict__ meta, int* __restrict__ tiles, int* __restrict__ ends) {
  __shared__ int count[MG_MAX_EXPERTS], offset[MG_MAX_EXPERTS], cursor[MG_MAX_EXPERTS];
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x)
    if (ids[i] < E) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < E; e++) {
      offset[e] = off;
      for (int r = 0; r < count[e]; r += MG_BM) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = off + r;
        tiles[3 * nt + 2] = min(MG_BM, count[e] - r);
        nt++;
      }
      off += count[e];
      if (ends) ends[e] = off;                 // where the expert's rows end: what a grouped library product reads
    }
    meta[0] = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= E) {                     // an identity expert: no row
      slot_of[i] = -1;
      continue;
    }
    const int row = offset[e] + atomicAdd(&cursor[e], 1);
    slot_of[i] = row;
    row_token[row] = i / top;
  }
  // rows that no pair took (pairs of identity experts have none) name token 0, so that a gather over all
  // n_pairs rows stays inside x
  const int used = offset[E - 1] + count[E - 1];
  for (int i = used + threadIdx.x; i < n_pairs; i += blockDim.x) row_token[i] = 0;
}

MF_API int mf_moe_sort(const int* ids, int T, int E, int top, int* slot_of, int* row_token, int* meta, int* tiles,
                       int* ends, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > MG_MAX_EXPERTS) return MF_ERR_BAD_ARG;
  mf_count(MF_K_MOE_SORT);
  moe_sort_kernel<<<1, 1024, 0, stream>>>(ids, T * top, E, top, slot_of, row_token, meta, tiles, ends);
  return (int)cudaGetLastError();
}

__device__ __forceinline__ void mg_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mg_cp16(void* smem, const void* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem) : "memory");
}

// One 64 x 64 tile: acc += A[64 rows, K] * B[64 rows of W, K]^T, A rows given by pointers.
// `arow(r)` -> pointer to row r of A (or null), `brow(n)` -> pointer to row n of W (or null).
// As: [MG_STAGES][64][MG_LD], Bs: [MG_STAGES][NB * 64][MG_LD].
template <int NB, typename ARow, typename BRow>
__device__ __forceinline__ void mg_tile(float (&acc)[NB][MG_BN / 8][4], int K, ARow arow, BRow brow,
                                        __nv_bfloat16* As, __nv_bfloat16* Bs) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto load = [&](int k0, int stage) {
    __nv_bfloat16* Ad = As + (size_t)stage * MG_BM * MG_LD;
    __nv_bfloat16* Bd = Bs + (size_t)stage * NB * MG_BN * MG_LD;
    for (int i = tid; i < MG_BM * (MG_BK / 8); i += blockDim.x) {
      const int r = i / (MG_BK / 8), c = (i - r * (MG_BK / 8)) * 8;
      const __nv_bfloat16* p = arow(r);
      if (p && k0 + c < K) mg_cp16(Ad + r * MG_LD + c, p + k0 + c);
      else *reinterpret_cast<uint4*>(Ad + r * MG_LD + c) = make_uint4(0, 0, 0, 0);
    }
    for (int i = tid; i < NB * MG_BN * (MG_BK / 8); i += blockDim.x) {
      const int n = i / (MG_BK / 8), c = (i - n * (MG_BK / 8)) * 8;
      const __nv_bfloat16* p = brow(n);
      if (p && k0 + c < K) mg_cp16(Bd + n * MG_LD + c, p + k0 + c);
      else *reinterpret_cast<uint4*>(Bd + n * MG_LD + c) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  load(0, 0);
  int stage = 0;
  for (int k0 = 0; k0 < K; k0 += MG_BK, stage ^= 1) {
    if (k0 + MG_BK < K) {
      load(k0 + MG_BK, stage ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* Ac = As + (size_t)stage * MG_BM * MG_LD;
    const __nv_bfloat16* Bc = Bs + (size_t)stage * NB * MG_BN * MG_LD;
#pragma unroll
    for (int kk = 0; kk < MG_BK; kk += 16) {
      // fragments by ldmatrix: A's four 8x8 blocks in one load, B's blocks of two column tiles in one
      uint32_t af[4];
      mg_ldmatrix_x4(af, Ac + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * MG_LD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int b = 0; b < NB; b++) {
#pragma unroll
        for (int nt = 0; nt < MG_BN / 8; nt += 2) {
          uint32_t bf[4];
          mg_ldmatrix_x4(bf, Bc + (b * MG_BN + nt * 8 + (lane & 7) + (lane >> 4) * 8) * MG_LD + kk + ((lane >> 3) & 1) * 8);
          mg_mma(acc[b][nt], af, bf[0], bf[1]);
          mg_mma(acc[b][nt + 1], af, bf[2], bf[3]);
        }
      }
    }
    __syncthreads();       // the stage is read: the load after the next may overwrite it
  }
}

// NB 2: gate and up tiles side by side and the gated activation; NB 1: an expert without a gate, whose
// first matrix is [ff, H] alone, and the activation `act_kind` of its sums.
template <int NB>
__global__ void __launch_bounds__(128)
moe_grouped_up_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_gu,
                      const int* __restrict__ row_token, const int* __restrict__ meta, const int* __restrict__ tiles,
                      __nv_bfloat16* __restrict__ act, int H, int ff, float limit, float alpha, float up_off,
                      int act_kind) {
  extern __shared__ __align__(16) __nv_bfloat16 mg_smem[];
  __nv_bfloat16* As = mg_smem;
  __nv_bfloat16* Bs = mg_smem + MG_STAGES * MG_BM * MG_LD;
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[3 * blockIdx.x], row_first = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * MG_BN;
  const __nv_bfloat16* wg = w_gu + (long long)e * NB * ff * H;
  const __nv_bfloat16* wu = wg + (long long)ff * H;
  float acc[NB][MG_BN / 8][4];
#pragma unroll
  for (int b = 0; b < NB; b++)
#pragma unroll
    for (int nt = 0; nt < MG_BN / 8; nt++) acc[b][nt][0] = acc[b][nt][1] = acc[b][nt][2] = acc[b][nt][3] = 0.f;
  mg_tile<NB>(acc, H,
             [&](int r) { return r < rows ? x + (long long)row_token[row_first + r] * H : nullptr; },
             [&](int n) {
               const int col = n0 + (n & (MG_BN - 1));
               if (col >= ff) return (const __nv_bfloat16*)nullptr;
               return (n < MG_BN ? wg : wu) + (long long)col * H;
             },
             As, Bs);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = warp * 16 + (lane >> 2), c2 = (lane & 3) * 2;
#pragma unroll
  for (int nt = 0; nt < MG_BN / 8; nt++) {
    const int col = n0 + nt * 8 + c2;
    if (col >= ff) continue;
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const int r = r0 + half * 8;
      if (r >= rows) continue;
      float v[2];
#pragma unroll
      for (int j = 0; j < 2; j++) {
        if (NB == 1) {
          v[j] = gate_act(acc[0][nt][half * 2 + j], act_kind);
          continue;
        }
        const float g = fminf(acc[0][nt][half * 2 + j], limit);
        const float u = fminf(fmaxf(acc[NB - 1][nt][half * 2 + j], -limit), limit);
        v[j] = g * (1.0f / (1.0f + __expf(-alpha * g))) * (u + up_off);
      }
      *reinterpret_cast<__nv_bfloat162*>(act + (long long)(row_first + r) * ff + col) = __floats2bfloat162_rn(v[0], v[1]);
    }
  }
}

__global__ void __launch_bounds__(128)
moe_grouped_down_kernel(const __nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ w_down,
                        const int* __restrict__ meta, const int* __restrict__ tiles, float* __restrict__ y, int H,
                        int ff) {
  extern __shared__ __align__(16) __nv_bfloat16 mg_smem[];
  __nv_bfloat16* As = mg_smem;
  __nv_bfloat16* Bs = mg_smem + MG_STAGES * MG_BM * MG_LD;
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[3 * blockIdx.x], row_first = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * MG_BN;
  const __nv_bfloat16* wd = w_down + (long long)e * H * ff;
  float acc[1][MG_BN / 8][4];
#pragma unroll
  for (int nt = 0; nt < MG_BN / 8; nt++) acc[0][nt][0] = acc[0][nt][1] = acc[0][nt][2] = acc[0][nt][3] = 0.f;
  mg_tile<1>(acc, ff,
             [&](int r) { return r < rows ? act + (long long)(row_first + r) * ff : nullptr; },
             [&](int n) { return n0 + n < H ? wd + (long long)(n0 + n) * ff : nullptr; }, As, Bs);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = warp * 16 + (lane >> 2), c2 = (lane & 3) * 2;
#pragma unroll
  for (int nt = 0; nt < MG_BN / 8; nt++) {
    const int col = n0 + nt * 8 + c2;
    if (col >= H) continue;
    if (r0 < rows) *reinterpret_cast<float2*>(y + (long long)(row_first + r0) * H + col) = make_float2(acc[0][nt][0], acc[0][nt][1]);
    if (r0 + 8 < rows)
      *reinterpret_cast<float2*>(y + (long long)(row_first + r0 + 8) * H + col) = make_float2(acc[0][nt][2], acc[0][nt][3]);
  }
}

// the kernels read rows in 16-byte pieces and write pairs of columns
MF_API int mf_moe_grouped_ok(int H, int ff, int E) {
  return (H % 8 == 0 && ff % 8 == 0 && E >= 1 && E <= MG_MAX_EXPERTS) ? 1 : 0;
}

// tiles the launches must cover for T tokens with `top` choices each among E experts
MF_API int mf_moe_grouped_max_tiles(int T, int top, int E) { return (T * top + MG_BM - 1) / MG_BM + E; }

MF_API int mf_moe_grouped_up(const void* x, const void* w_gu, const int* row_token, const int* meta, const int* tiles,
                             void* act, int T, int H, int ff, int E, int top, float limit, float alpha, float up_off,
                             int act_kind, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!mf_moe_grouped_ok(H, ff, E)) return MF_ERR_BAD_ARG;
  dim3 grid(mf_moe_grouped_max_tiles(T, top, E), (ff + MG_BN - 1) / MG_BN);
  mf_count(MF_K_MOE_GROUPED);
  const size_t smem = (size_t)MG_STAGES * (MG_BM + 2 * MG_BN) * MG_LD * sizeof(__nv_bfloat16);
  static DeviceOnce once;
  const int dev = mf_current_device();
  if (dev < 0 || act_kind >= MF_ACT_COUNT) return MF_ERR_BAD_ARG;
  if (!once.done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_up_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(moe_grouped_up_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    once.done[dev] = true;
  }
  if (act_kind < 0)
    moe_grouped_up_kernel<2><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gu, row_token,
                                                          meta, tiles, (__nv_bfloat16*)act, H, ff, limit, alpha, up_off,
                                                          act_kind);
  else
    moe_grouped_up_kernel<1><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gu, row_token,
                                                          meta, tiles, (__nv_bfloat16*)act, H, ff, limit, alpha, up_off,
                                                          act_kind);
  return (int)cudaGetLastError();
}

MF_API int mf_moe_grouped_down(const void* act, const void* w_down, const int* meta, const int* tiles, float* y, int T,
                               int H, int ff, int E, int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!mf_moe_grouped_ok(H, ff, E)) return MF_ERR_BAD_ARG;
  dim3 grid(mf_moe_grouped_max_tiles(T, top, E), (H + MG_BN - 1) / MG_BN);
  mf_count(MF_K_MOE_GROUPED);
  const size_t smem = (size_t)MG_STAGES * (MG_BM + MG_BN) * MG_LD * sizeof(__nv_bfloat16);
  moe_grouped_down_kernel<<<grid, 128, smem, stream>>>((const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, meta, tiles,
                                                    y, H, ff);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ around the library's grouped product
// xg[row] = x[row_token[row]], 16 bytes a copy (H a multiple of 8)
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ row_token, uint4* __restrict__ xg, int h8) {
  const long long row = blockIdx.x;
  const uint4* src = x + (long long)row_token[row] * h8;
  for (int i = threadIdx.x; i < h8; i += blockDim.x) xg[row * h8 + i] = src[i];
}

MF_API int mf_moe_gather_rows(const void* x, const int* row_token, void* xg, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (H % 8) return MF_ERR_BAD_ARG;
  mf_count(MF_K_MOE_GROUPED);
  moe_gather_rows_kernel<<<n_rows, 256, 0, stream>>>((const uint4*)x, row_token, (uint4*)xg, H / 8);
  return (int)cudaGetLastError();
}

// act[r, f] = g sigmoid(alpha g) (u + up_off), g = min(gu[r, f], limit), u = clamp(gu[r, ff + f], -limit, limit)
__global__ void __launch_bounds__(256)
moe_activation_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int ff, float limit,
                      float alpha, float up_off, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long r = i / ff;
  const int f = (int)(i - r * ff);
  const float g = fminf(__bfloat162float(gu[r * 2 * ff + f]), limit);
  const float u = fminf(fmaxf(__bfloat162float(gu[r * 2 * ff + ff + f]), -limit), limit);
  act[i] = __float2bfloat16_rn(g * (1.0f / (1.0f + __expf(-alpha * g))) * (u + up_off));
}

// the same, 8 columns a thread (ff a multiple of 8)
__global__ void __launch_bounds__(256)
moe_activation_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int ff, float limit,
                          float alpha, float up_off, long long total8) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  const int f8 = ff / 8;
  const long long r = i / f8;
  const int f = (int)(i - r * f8) * 8;
  const uint4 gv = *reinterpret_cast<const uint4*>(gu + r * 2 * ff + f);
  const uint4 uv = *reinterpret_cast<const uint4*>(gu + r * 2 * ff + ff + f);
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const float2 g2 = __bfloat1622float2(gp[j]), u2 = __bfloat1622float2(up[j]);
    const float g0 = fminf(g2.x, limit), g1 = fminf(g2.y, limit);
    const float u0 = fminf(fmaxf(u2.x, -limit), limit), u1 = fminf(fmaxf(u2.y, -limit), limit);
    op[j] = __floats2bfloat162_rn(g0 * (1.0f / (1.0f + __expf(-alpha * g0))) * (u0 + up_off),
                                  g1 * (1.0f / (1.0f + __expf(-alpha * g1))) * (u1 + up_off));
  }
  *reinterpret_cast<uint4*>(act + r * ff + f) = o;
}

MF_API int mf_moe_activation(const void* gu, void* act, int n_rows, int ff, float limit, float alpha, float up_off,
                             cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const long long total = (long long)n_rows * ff;
  mf_count(MF_K_MOE_GROUPED);
  if (ff % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)act & 15) == 0) {
    const long long total8 = total / 8;
    moe_activation_vec_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, ff, limit, alpha, up_off, total8);
    return (int)cudaGetLastError();
  }
  moe_activation_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)gu,
                                                                             (__nv_bfloat16*)act, ff, limit, alpha, up_off, total);
  return (int)cudaGetLastError();
}
