// Routed experts: every token goes through the `top` experts its router picks.
//
//   mi_moe_route      z = W_r x in fp32; the `top` largest logits of a token (ties: the lower index) and
//                     the softmax over those alone -> ids [M, top] int32, weights [M, top] fp32
//   mi_moe_plan       sorts the M*top (token, choice) entries by expert: perm[pos] = entry, inv[entry] =
//                     pos, offsets[E + 1], and the list of row tiles (expert, first row, rows) that the
//                     grouped products walk.  Nothing comes back to the host: the products are launched
//                     for the largest possible number of tiles and the surplus blocks leave at once.
//   mi_moe_gate_up    act[pos, :] = glu(W_gate[e] x_token, W_up[e] x_token) for the entries of each expert
//   mi_moe_down       y[pos, :] = W_down[e] act[pos, :]   (fp32)
//   mi_moe_combine    out[t, :] = T(sum_k weight[t, k] * y[inv[t*top + k], :] + shared[t, :])
//   mi_clamped_glu    the same activation for a dense expert: out = glu(gu[:, :I], gu[:, I:])
//
// glu(g, u) = g' * sigmoid(alpha * g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit).
//
// The products run on CUDA cores with fp32 accumulation, k ascending, so a row's result does not
// depend on which other rows share its tile.
#include "common.cuh"

MI_DEFINE_ERROR_API()

__device__ __forceinline__ float mi_clamped_glu_value(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.f / (1.f + expf(-alpha * g))) * (u + 1.f);
}

// ------------------------------------------------------------------------------------------ router
#define ROUTE_MAX_PER_LANE 8

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ wr,
                                 int* __restrict__ ids, float* __restrict__ weights, int M, int H, int E, int top) {
  mi_pdl_enter();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= M) return;
  const T* xr = x + (size_t)t * x_stride;
  float lg[ROUTE_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) lg[i] = -INFINITY;
  for (int e = 0; e < E; ++e) {
    const T* w = wr + (size_t)e * H;
    float acc = 0.f;
    for (int h = lane; h < H; h += 32) acc = fmaf(mi_to_float(xr[h]), mi_to_float(w[h]), acc);
    acc = mi_warp_sum(acc);
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
      if (e == lane + 32 * i) lg[i] = acc;
  }
  float my_val = 0.f, denom = 0.f, first = 0.f;
  int my_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (lg[i] > best || (lg[i] == best && e < best_e)) && lg[i] != -INFINITY) {
        best = lg[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
      if (best_e == lane + 32 * i) lg[i] = -INFINITY;   // taken
    if (k == 0) first = best;
    const float p = expf(best - first);
    denom += p;
    if (lane == k) {
      my_val = p;
      my_id = best_e;
    }
  }
  if (lane < top) {
    ids[(size_t)t * top + lane] = my_id;
    weights[(size_t)t * top + lane] = my_val / denom;
  }
}

extern "C" int mi_moe_route(const void* x, int x_stride, const void* wr, int* ids, float* weights, int M, int H,
                            int E, int top, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > 32 * ROUTE_MAX_PER_LANE) MI_REFUSE("moe: %d experts (1 to %d are taken)", E, 32 * ROUTE_MAX_PER_LANE);
  if (top <= 0 || top > E || top > 32) MI_REFUSE("moe: %d of %d experts per token", top, E);
  const int blocks = (M + 3) / 4;
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_route_kernel<float>), blocks, 128, 0, stream, (const float*)x, x_stride, (const float*)wr, ids,
              weights, M, H, E, top);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_route_kernel<bf16>), blocks, 128, 0, stream, (const bf16*)x, x_stride, (const bf16*)wr, ids,
              weights, M, H, E, top);
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ plan
#define TILE_M 64
#define TILE_N 64
#define TILE_K 16

// plan layout (int32): [0] number of tiles, [1 .. E+1] offsets, then 3 ints per tile (expert, first row, rows)
__global__ void moe_plan_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ perm,
                                int* __restrict__ inv, int* __restrict__ plan) {
  mi_pdl_enter();
  extern __shared__ int sh[];
  int* counts = sh;            // [E]
  int* cursor = sh + E;        // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int* offsets = plan + 1;
    int* tiles = plan + 2 + E;
    int run = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      const int end = run + counts[e];
      for (int r0 = run; r0 < end; r0 += TILE_M) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = r0;
        tiles[3 * nt + 2] = min(TILE_M, end - r0);
        ++nt;
      }
      run = end;
    }
    offsets[E] = run;
    plan[0] = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int pos = atomicAdd(&cursor[ids[i]], 1);
    perm[pos] = i;
    inv[i] = pos;
  }
}

extern "C" int mi_moe_tile_rows() { return TILE_M; }

extern "C" int mi_moe_plan(const int* ids, int n, int E, int* perm, int* inv, int* plan, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E <= 0 || E > 4096) MI_REFUSE("moe: %d experts", E);
  MI_LAUNCH((moe_plan_kernel), 1, 1024, 2 * E * sizeof(int), stream, ids, n, E, perm, inv, plan);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ grouped products
// A tile is TILE_M rows of one expert times TILE_N output columns; 256 threads, 4 x 4 outputs each.
// GATED: A rows are gathered (token = perm[pos] / top), two weight matrices, the activation in the
// epilogue, output in T.  Otherwise A rows are the sorted rows themselves and the output is fp32.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ a, int a_stride, const T* __restrict__ w0, const T* __restrict__ w1,
                long long w_expert_stride, const int* __restrict__ perm, int top, const int* __restrict__ plan,
                int E, void* __restrict__ out_, int N, int K, float limit, float alpha) {
  mi_pdl_enter();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* td = plan + 2 + E + 3 * tile;
  const int e = td[0], row0 = td[1], rows = td[2];
  const int n0 = blockIdx.x * TILE_N;
  __shared__ float As[TILE_K][TILE_M + 4];
  __shared__ float B0[TILE_K][TILE_N + 4];
  __shared__ float B1[GATED ? TILE_K : 1][TILE_N + 4];
  __shared__ int arow[TILE_M];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < TILE_M) {
    int r = -1;
    if (tid < rows) r = GATED ? perm[row0 + tid] / top : row0 + tid;
    arow[tid] = r;
  }
  const T* wb0 = w0 + (size_t)e * w_expert_stride;
  const T* wb1 = GATED ? w1 + (size_t)e * w_expert_stride : nullptr;
  float acc0[4][4], acc1[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc0[i][j] = acc1[i][j] = 0.f;
  __syncthreads();
  for (int k0 = 0; k0 < K; k0 += TILE_K) {
    // 64 x 16 elements of each operand: 4 per thread, k fastest
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + 256 * it;
      const int r = idx >> 4, kk = idx & 15;
      const int kg = k0 + kk;
      const int ar = arow[r];
      As[kk][r] = (ar >= 0 && kg < K) ? mi_to_float(a[(size_t)ar * a_stride + kg]) : 0.f;
      const int n = n0 + r;
      const bool ok = n < N && kg < K;
      B0[kk][r] = ok ? mi_to_float(wb0[(size_t)n * K + kg]) : 0.f;
      if (GATED) B1[kk][r] = ok ? mi_to_float(wb1[(size_t)n * K + kg]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TILE_K; ++kk) {
      float av[4], b0[4], b1[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b0[j] = B0[kk][tx * 4 + j];
        if (GATED) b1[j] = B1[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc0[i][j] = fmaf(av[i], b0[j], acc0[i][j]);
          if (GATED) acc1[i][j] = fmaf(av[i], b1[j], acc1[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (GATED)
        reinterpret_cast<T*>(out_)[(size_t)(row0 + r) * N + n] =
            mi_from_float<T>(mi_clamped_glu_value(acc0[i][j], acc1[i][j], limit, alpha));
      else
        reinterpret_cast<float*>(out_)[(size_t)(row0 + r) * N + n] = acc0[i][j];
    }
  }
}

static int max_tiles(int n_entries, int E) { return (n_entries + TILE_M - 1) / TILE_M + E; }

extern "C" int mi_moe_gate_up(const void* x, int x_stride, const void* w_gate, const void* w_up,
                              long long w_expert_stride, const int* perm, int top, const int* plan, int E,
                              void* act, int n_entries, int ff, int H, float limit, float alpha, int dtype,
                              cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  dim3 grid((ff + TILE_N - 1) / TILE_N, max_tiles(n_entries, E));
  if (grid.y > 65535) MI_REFUSE("moe: too many row tiles for one launch");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_gemm_kernel<float, true>), grid, 256, 0, stream, (const float*)x, x_stride, (const float*)w_gate,
              (const float*)w_up, w_expert_stride, perm, top, plan, E, act, ff, H, limit, alpha);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_gemm_kernel<bf16, true>), grid, 256, 0, stream, (const bf16*)x, x_stride, (const bf16*)w_gate,
              (const bf16*)w_up, w_expert_stride, perm, top, plan, E, act, ff, H, limit, alpha);
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

extern "C" int mi_moe_down(const void* act, const void* w_down, long long w_expert_stride, const int* plan, int E,
                           float* y, int n_entries, int H, int ff, int dtype, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  dim3 grid((H + TILE_N - 1) / TILE_N, max_tiles(n_entries, E));
  if (grid.y > 65535) MI_REFUSE("moe: too many row tiles for one launch");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_gemm_kernel<float, false>), grid, 256, 0, stream, (const float*)act, ff, (const float*)w_down,
              (const float*)nullptr, w_expert_stride, (const int*)nullptr, 1, plan, E, (void*)y, H, ff, 0.f, 0.f);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_gemm_kernel<bf16, false>), grid, 256, 0, stream, (const bf16*)act, ff, (const bf16*)w_down,
              (const bf16*)nullptr, w_expert_stride, (const int*)nullptr, 1, plan, E, (void*)y, H, ff, 0.f, 0.f);
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ combine
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ inv,
                                   const float* __restrict__ weights, const T* __restrict__ shared, int shared_stride,
                                   T* __restrict__ out, int H, int top) {
  mi_pdl_enter();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(weights[(size_t)t * top + k], y[(size_t)inv[(size_t)t * top + k] * H + c], acc);
    if (shared) acc += mi_to_float(shared[(size_t)t * shared_stride + c]);
    out[(size_t)t * H + c] = mi_from_float<T>(acc);
  }
}

extern "C" int mi_moe_combine(const float* y, const int* inv, const float* weights, const void* shared,
                              int shared_stride, void* out, int M, int H, int top, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_combine_kernel<float>), M, threads, 0, stream, y, inv, weights, (const float*)shared,
              shared_stride, (float*)out, H, top);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_combine_kernel<bf16>), M, threads, 0, stream, y, inv, weights, (const bf16*)shared,
              shared_stride, (bf16*)out, H, top);
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ dense expert
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, int stride, T* __restrict__ out, int M, int I,
                                   float limit, float alpha) {
  mi_pdl_enter();
  const size_t n = (size_t)M * I;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / I), c = (int)(idx - (size_t)t * I);
    const float g = mi_to_float(gu[(size_t)t * stride + c]), u = mi_to_float(gu[(size_t)t * stride + I + c]);
    out[idx] = mi_from_float<T>(mi_clamped_glu_value(g, u, limit, alpha));
  }
}

extern "C" int mi_clamped_glu(const void* gu, int stride, void* out, int M, int I, float limit, float alpha,
                              int dtype, cudaStream_t stream) {
  if (M <= 0 || I <= 0) return 0;
  const size_t n = (size_t)M * I;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((clamped_glu_kernel<float>), blocks, 256, 0, stream, (const float*)gu, stride, (float*)out, M, I, limit, alpha);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((clamped_glu_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)gu, stride, (bf16*)out, M, I, limit, alpha);
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}
