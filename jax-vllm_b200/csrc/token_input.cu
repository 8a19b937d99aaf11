// The gate of a per-layer token input:  g[t, j] = gelu_tanh(z[t, j]) * table[token[t], offset + j],
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), in 32-bit; z is the product gate(x), which the
// caller keeps in 32-bit (far in its negative tail the activation is a small difference of z's digits).
#include "common.cuh"
#include <math.h>

namespace {
template <typename TZ, typename T, typename TE>
__global__ void token_gate_kernel(const TZ* __restrict__ z, const int* __restrict__ tokens, const TE* __restrict__ table,
                                  int table_width, int offset, int vocab, T* __restrict__ g, int n, int dim,
                                  int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n * dim;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / dim;
    const int j = (int)(i - t * dim);
    const int id = tokens[t];
    float e = 0.f;
    if (id < 0 || id >= vocab) {
      if (j == 0) atomicOr(status, JV_STATUS_BAD_TOKEN);
    } else {
      e = to_f32(table[(size_t)id * table_width + offset + j]);
    }
    const float v = to_f32(z[i]);
    const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    g[i] = from_f32<T>(0.5f * v * (1.f + tanhf(u)) * e);
  }
}
}  // namespace

// z: [n, dim] of `z_dtype`; g: [n, dim] of `dtype`; tokens: [n] int32; table: [vocab, table_width] of `table_dtype`.
JV_EXPORT int jv_token_gate(const void* z, int z_dtype, int dtype, const int* tokens, const void* table, int table_dtype,
                            int table_width, int offset, int vocab, void* g, int n, int dim, int* status,
                            cudaStream_t stream) {
  if (n == 0) return JV_OK;
  long long blocks = ((long long)n * dim + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  JV_DISPATCH_DTYPE(z_dtype, TZ, JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(table_dtype, TE,
      return jv_launch(token_gate_kernel<TZ, T, TE>, dim3((int)blocks), dim3(256), 0, stream, (const TZ*)z, tokens,
                       (const TE*)table, table_width, offset, vocab, (T*)g, n, dim, status))));
  return JV_ERR_UNSUPPORTED;
}
