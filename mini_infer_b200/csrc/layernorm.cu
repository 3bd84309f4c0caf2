// Layer norm over the fp32 residual stream, and the scaled token embedding that starts it.
//
//   mi_embedding_scaled   stream[t, :] = float(table[ids[t], :]) * scale          (fp32 out)
//   mi_add_layernorm      r = stream[src] + float(add1[src]) + float(add2[src])   (fp32)
//                         stream_out[i] = r                       (if given; may be the stream itself)
//                         out1[i] = T((r - mean) * rstd * w1 + b1)
//                         out2[i] = T((r - mean) * rstd * w2 + b2)   (if given: a second norm of the
//                                   same row, for layers whose two branches read the same stream)
//
// mean and variance are fp32, the variance is the mean of the squared deviations (two passes
// over the row, which is kept in shared memory).  One block per output row; src = rows[i] when a
// gather list is given, else i.  Gains and biases are fp32.
#include "common.cuh"

MI_DEFINE_ERROR_API()

template <typename T>
__global__ void embedding_scaled_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                        float* __restrict__ out, int H, int V, float scale) {
  mi_pdl_enter();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (size_t)t * H;
  if ((unsigned)id >= (unsigned)V) {   // the step function validates ids; this keeps a fault visible
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __int_as_float(0x7fc00000);
    return;
  }
  const T* src = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = mi_to_float(src[i]) * scale;
}

extern "C" int mi_embedding_scaled(const void* table, const int* ids, float* out, int M, int H, int V,
                                   float scale, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0 || V <= 0) MI_REFUSE("embedding: bad sizes H=%d V=%d", H, V);
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((embedding_scaled_kernel<float>), M, threads, 0, stream, (const float*)table, ids, out, H, V, scale);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((embedding_scaled_kernel<bf16>), M, threads, 0, stream, (const bf16*)table, ids, out, H, V, scale);
  else
    MI_REFUSE("embedding: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

template <typename T>
__global__ void add_layernorm_kernel(const float* __restrict__ stream, const T* __restrict__ add1,
                                     const T* __restrict__ add2, float* __restrict__ stream_out,
                                     const int* __restrict__ rows, const float* __restrict__ w1,
                                     const float* __restrict__ b1, T* __restrict__ out1,
                                     const float* __restrict__ w2, const float* __restrict__ b2,
                                     T* __restrict__ out2, int H, float eps) {
  mi_pdl_enter();
  extern __shared__ float smem[];
  float* red = smem;        // 32 floats
  float* row = smem + 32;   // H floats
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  const float* sr = stream + (size_t)src * H;
  const T* a1 = add1 ? add1 + (size_t)src * H : nullptr;
  const T* a2 = add2 ? add2 + (size_t)src * H : nullptr;
  float sum = 0.f;
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    float r = sr[k];
    if (a1) r += mi_to_float(a1[k]);
    if (a2) r += mi_to_float(a2[k]);
    row[k] = r;
    sum += r;
  }
  const float mean = mi_block_sum(sum, red) / (float)H;
  float sq = 0.f;
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    const float dlt = row[k] - mean;
    sq += dlt * dlt;
  }
  const float rstd = 1.f / sqrtf(mi_block_sum(sq, red) / (float)H + eps);
  float* so = stream_out ? stream_out + (size_t)i * H : nullptr;
  T* o1 = out1 + (size_t)i * H;
  T* o2 = out2 ? out2 + (size_t)i * H : nullptr;
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    const float r = row[k];
    const float n = (r - mean) * rstd;
    if (so) so[k] = r;
    o1[k] = mi_from_float<T>(n * w1[k] + b1[k]);
    if (o2) o2[k] = mi_from_float<T>(n * w2[k] + b2[k]);
  }
}

extern "C" int mi_add_layernorm(const float* stream, const void* add1, const void* add2, float* stream_out,
                                const int* rows, const float* w1, const float* b1, void* out1,
                                const float* w2, const float* b2, void* out2, int M, int H, float eps,
                                int dtype, cudaStream_t stream_) {
  if (M <= 0) return 0;
  if (H <= 0) MI_REFUSE("layernorm: bad width %d", H);
  if (rows && stream_out == stream) MI_REFUSE("layernorm: a gathered norm cannot update the stream in place");
  const size_t smem = (32 + (size_t)H) * sizeof(float);
  if (smem > 200 * 1024) MI_REFUSE("layernorm: a row of %d floats does not fit in shared memory", H);
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define MI_GO(T)                                                                                       \
  do {                                                                                                 \
    auto kern = add_layernorm_kernel<T>;                                                               \
    if (smem > 48 * 1024) {                                                                            \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                             \
    }                                                                                                  \
    MI_LAUNCH(kern, M, threads, smem, stream_, stream, (const T*)add1, (const T*)add2, stream_out, rows, w1, b1, \
              (T*)out1, w2, b2, (T*)out2, H, eps);                                                     \
  } while (0)
  if (dtype == MI_DTYPE_F32) MI_GO(float);
  else if (dtype == MI_DTYPE_BF16) MI_GO(bf16);
  else MI_REFUSE("layernorm: unknown dtype %d", dtype);
#undef MI_GO
  MI_RETURN_LAUNCH_STATUS();
}
