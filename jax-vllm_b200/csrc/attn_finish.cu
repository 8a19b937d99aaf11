// What happens to attention heads between the attention kernel and the output projection, in one pass
// (one warp per token and head, 32-bit arithmetic):
//
//   two score maps on the same values (optional): the attention kernel ran 2*H heads, map 1 of head h at
//       index h, map 2 at H + h;  o = a1 - lambda * a2
//   unit norm over the head (optional): o <- o * rsqrt(mean(o^2) + eps) * post   (no weight)
//   gate (optional): o <- o * sigmoid(g), g one number per head (gate_kind 1, at gate[n, h]) or one per
//       element (gate_kind 2, at gate[n, h*DV + d]); the gate is a column range of the packed projection
//
// in: [n, maps*H, DV] float or the compute type; out: [n, out_stride] of the compute type, head h at h*DV.
#include "common.cuh"

namespace {
template <typename TI, typename T>
__global__ void attn_finish_kernel(const TI* __restrict__ in, T* __restrict__ out, long long out_stride,
                                   const T* __restrict__ gate, long long gate_stride, int gate_kind, int n, int heads,
                                   int dv, int maps, float lambda, int unit_norm, float eps, float post) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)n * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const TI* a1 = in + ((size_t)t * maps * heads + h) * dv;
  const TI* a2 = a1 + (size_t)heads * dv;
  float ss = 0.f;
  if (unit_norm) {
    for (int d = lane; d < dv; d += 32) {
      float o = to_f32(a1[d]);
      if (maps == 2) o -= lambda * to_f32(a2[d]);
      ss += o * o;
    }
    ss = warp_sum(ss);
  }
  const float mul = unit_norm ? rsqrtf(ss / (float)dv + eps) * post : post;
  float g_head = 1.f;
  if (gate_kind == 1) g_head = 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + h])));
  for (int d = lane; d < dv; d += 32) {
    float o = to_f32(a1[d]);
    if (maps == 2) o -= lambda * to_f32(a2[d]);
    o *= mul * g_head;
    if (gate_kind == 2) o *= 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + (size_t)h * dv + d])));
    out[(size_t)t * out_stride + (size_t)h * dv + d] = from_f32<T>(o);
  }
}
}  // namespace

// in_dtype / dtype: 0 = float, 1 = bfloat16 (in may be float while out and gate are bfloat16).
JV_EXPORT int jv_attn_finish(const void* in, int in_dtype, void* out, int dtype, long long out_stride, const void* gate,
                             long long gate_stride, int gate_kind, int n, int heads, int dv, int maps, float lambda,
                             int unit_norm, float eps, float post, cudaStream_t stream) {
  if (n == 0 || heads == 0) return JV_OK;
  if ((maps != 1 && maps != 2) || gate_kind < 0 || gate_kind > 2 || (gate_kind && gate == nullptr)) return JV_ERR_UNSUPPORTED;
  const int warps = 4;
  const long long items = (long long)n * heads;
  const dim3 grid((unsigned)((items + warps - 1) / warps));
  JV_DISPATCH_DTYPE(dtype, T, {
    if (in_dtype == 0)
      return jv_launch(attn_finish_kernel<float, T>, grid, dim3(32 * warps), 0, stream, (const float*)in, (T*)out,
                       out_stride, (const T*)gate, gate_stride, gate_kind, n, heads, dv, maps, lambda, unit_norm, eps, post);
    if (in_dtype == dtype)
      return jv_launch(attn_finish_kernel<T, T>, grid, dim3(32 * warps), 0, stream, (const T*)in, (T*)out,
                       out_stride, (const T*)gate, gate_stride, gate_kind, n, heads, dv, maps, lambda, unit_norm, eps, post);
  });
  return JV_ERR_UNSUPPORTED;
}
