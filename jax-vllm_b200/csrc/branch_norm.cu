// The residual update of a layer that norms each branch's OUTPUT:
//
//   h[r, :] += mult * b[r, :] * rsqrt(mean(b[r, :]^2) + eps) * weight[:]          (32-bit throughout)
//   x[r, :]  = h[r, :] rounded to the compute type                                (optional: what the next branch reads)
//
// The branch b comes in one of three forms, all summed in 32-bit in a fixed order:
//   * a tensor [n, hidden];
//   * `parts` tensors `part_stride` elements apart whose sum it is (a product whose k was cut);
//   * rows of a tensor picked per output row with a coefficient each: b[r] = sum_s coef[r, s] * y[pick[r, s]]
//     (the chosen experts' outputs of a routed feed-forward, weighted by their router scores), s ascending.
// The row of b is kept in shared memory between the two passes, so it is formed once.
#include "common.cuh"

namespace {
constexpr int MAX_PICKS = 64;     // rows that one row of a branch may be the weighted sum of

template <typename TD, typename TW, typename TX>
__global__ void branch_norm_add_kernel(float* __restrict__ h, const TD* __restrict__ y, size_t part_stride, int parts,
                                       const int* __restrict__ pick, const float* __restrict__ coef, int y_rows,
                                       const TW* __restrict__ weight, TX* __restrict__ x_out, int hidden, float eps,
                                       float mult, int* __restrict__ status) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  __shared__ int pick_s[MAX_PICKS];
  __shared__ float coef_s[MAX_PICKS];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (pick != nullptr) {
    // which rows, and their weights, once for the block; a row outside the tensor is left out (and reported)
    if (threadIdx.x < parts) {
      int src = pick[(size_t)r * parts + threadIdx.x];
      if (src < 0 || src >= y_rows) { atomicOr(status, JV_STATUS_BAD_ROW); src = -1; }
      pick_s[threadIdx.x] = src;
      coef_s[threadIdx.x] = coef[(size_t)r * parts + threadIdx.x];
    }
    __syncthreads();
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = 0.f;
    if (pick != nullptr) {
      for (int s = 0; s < parts; ++s)
        if (pick_s[s] >= 0) v = fmaf(coef_s[s], to_f32(y[(size_t)pick_s[s] * hidden + c]), v);
    } else {
      v = to_f32(y[(size_t)r * hidden + c]);
      for (int s = 1; s < parts; ++s) v += to_f32(y[s * part_stride + (size_t)r * hidden + c]);
    }
    row[c] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = mult * rsqrtf(ss / (float)hidden + eps);
  float* hr = h + (size_t)r * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = hr[c] + row[c] * inv * to_f32(weight[c]);
    hr[c] = v;
    if (x_out != nullptr) x_out[(size_t)r * hidden + c] = from_f32<TX>(v);
  }
}

// eight elements at a time (16 bytes of bfloat16, 32 of float)
template <typename T> __device__ __forceinline__ void ld8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void ld8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void st8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void st8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 a;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = a;
}

// The same as branch_norm_add_kernel with eight elements a thread and pass (hidden a multiple of 8, every pointer
// 16-byte aligned): the sums are formed in the same order, element by element, so the results are the same bits.
template <typename TD, typename TW, typename TX>
__global__ void branch_norm_add_vec_kernel(float* __restrict__ h, const TD* __restrict__ y, size_t part_stride, int parts,
                                           const int* __restrict__ pick, const float* __restrict__ coef, int y_rows,
                                           const TW* __restrict__ weight, TX* __restrict__ x_out, int hidden, float eps,
                                           float mult, int* __restrict__ status) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  __shared__ int pick_s[MAX_PICKS];
  __shared__ float coef_s[MAX_PICKS];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (pick != nullptr) {
    if (threadIdx.x < parts) {
      int src = pick[(size_t)r * parts + threadIdx.x];
      if (src < 0 || src >= y_rows) { atomicOr(status, JV_STATUS_BAD_ROW); src = -1; }
      pick_s[threadIdx.x] = src;
      coef_s[threadIdx.x] = coef[(size_t)r * parts + threadIdx.x];
    }
    __syncthreads();
  }
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float v[8];
    if (pick != nullptr) {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = 0.f;
      for (int s = 0; s < parts; ++s)
        if (pick_s[s] >= 0) {
          float t[8];
          ld8<TD>(y + (size_t)pick_s[s] * hidden + c, t);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = fmaf(coef_s[s], t[k], v[k]);
        }
    } else {
      ld8<TD>(y + (size_t)r * hidden + c, v);
      for (int s = 1; s < parts; ++s) {
        float t[8];
        ld8<TD>(y + s * part_stride + (size_t)r * hidden + c, t);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] += t[k];
      }
    }
    st8<float>(row + c, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
  }
  ss = block_sum(ss, scratch);
  const float inv = mult * rsqrtf(ss / (float)hidden + eps);
  float* hr = h + (size_t)r * hidden;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float a[8], b[8], w[8];
    ld8<float>(hr + c, a);
    ld8<float>(row + c, b);
    ld8<TW>(weight + c, w);
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = a[k] + b[k] * inv * w[k];
    st8<float>(hr + c, a);
    if (x_out != nullptr) st8<TX>(x_out + (size_t)r * hidden + c, a);
  }
}

template <typename TD>
__global__ void pick_rows_sum_kernel(const TD* __restrict__ y, const int* __restrict__ pick, const float* __restrict__ coef,
                                     int parts, int y_rows, float* __restrict__ out, int hidden, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < parts; ++s) {
      const int src = pick[(size_t)r * parts + s];
      if (src < 0 || src >= y_rows) {
        if (c == 0) atomicOr(status, JV_STATUS_BAD_ROW);
        continue;
      }
      v = fmaf(coef[(size_t)r * parts + s], to_f32(y[(size_t)src * hidden + c]), v);
    }
    out[(size_t)r * hidden + c] = v;
  }
}

template <typename TX>
__global__ void cast_rows_kernel(const float* __restrict__ h, TX* __restrict__ x, size_t n) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] = from_f32<TX>(h[i]);
}
}  // namespace

// h: [n, hidden] float, updated in place.  y: the branch, of dtype `y_dtype`: [n, hidden]; or `parts` such
// tensors `part_stride` elements apart (pick null); or [y_rows, hidden] with pick [n, parts] int32 rows of it and
// coef [n, parts] float.  weight: [hidden] of `weight_dtype`.  x_out: [n, hidden] of `x_dtype`, or null.
JV_EXPORT int jv_branch_norm_add(float* h, const void* y, int y_dtype, long long part_stride, int parts,
                                 const int* pick, const float* coef, int y_rows, const void* weight,
                                 int weight_dtype, void* x_out, int x_dtype, int n, int hidden, float eps, float mult,
                                 int* status, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (parts < 1 || (pick != nullptr && parts > MAX_PICKS) || (size_t)hidden * sizeof(float) > 200 * 1024) return JV_ERR_UNSUPPORTED;
  int threads = 64;
  while (threads < 512 && threads * 4 < hidden) threads *= 2;
  const size_t smem = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 8 == 0 && part_stride % 8 == 0 && ((uintptr_t)h % 16) == 0 && ((uintptr_t)y % 16) == 0 &&
                   ((uintptr_t)weight % 16) == 0 && ((uintptr_t)x_out % 16) == 0;
  if (vec) {
    threads = 32;
    while (threads < 256 && threads * 8 < hidden) threads *= 2;
  }
  JV_DISPATCH_DTYPE(y_dtype, TD, JV_DISPATCH_DTYPE(weight_dtype, TW, JV_DISPATCH_DTYPE(x_dtype, TX, {
    auto kern = vec ? branch_norm_add_vec_kernel<TD, TW, TX> : branch_norm_add_kernel<TD, TW, TX>;
    if (smem > 48 * 1024) {       // rows beyond 12,288 elements: both forms are allowed the larger size once
      static size_t allowed = 0;
      if (smem > allowed) {
        if (cudaFuncSetAttribute(branch_norm_add_vec_kernel<TD, TW, TX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(branch_norm_add_kernel<TD, TW, TX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
          return JV_ERR_UNSUPPORTED;
        allowed = smem;
      }
    }
    return jv_launch(kern, dim3(n), dim3(threads), smem, stream, h, (const TD*)y, (size_t)part_stride, parts, pick,
                     coef, y_rows, (const TW*)weight, (TX*)x_out, hidden, eps, mult, status);
  })));
  return JV_ERR_UNSUPPORTED;
}

// out[r, :] = sum_s coef[r, s] * y[pick[r, s], :] in 32-bit, s ascending: the weighted rows added up for a reader
// that does not add them itself.
JV_EXPORT int jv_pick_rows_sum(const void* y, int y_dtype, const int* pick, const float* coef, int parts, int y_rows,
                               float* out, int n, int hidden, int* status, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  JV_DISPATCH_DTYPE(y_dtype, TD, return jv_launch(pick_rows_sum_kernel<TD>, dim3(n), dim3(256), 0, stream, (const TD*)y,
                                                  pick, coef, parts, y_rows, out, hidden, status));
  return JV_ERR_UNSUPPORTED;
}

// x = h rounded to `x_dtype` (n elements).
JV_EXPORT int jv_cast_rows(const float* h, void* x, int x_dtype, long long n, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  JV_DISPATCH_DTYPE(x_dtype, TX, return jv_launch(cast_rows_kernel<TX>, dim3((int)blocks), dim3(256), 0, stream, h,
                                                  (TX*)x, (size_t)n));
  return JV_ERR_UNSUPPORTED;
}
