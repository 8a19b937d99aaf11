// Query/key/value preparation for attention mixers whose heads are not all alike, fused with the
// write of the new keys and values into the paged cache.  A few blocks handle one token of a packed
// projection row `proj` (queries at q_off, keys at k_off, values at v_off; element offsets):
//
//   whole-projection RMSNorm (optional, queries and keys separately): all heads of a token form ONE
//       vector u of Hq*D (Hk*D) elements, u <- u * rsqrt(mean(u^2) + eps) * weight[Hq*D]
//   query temperature (optional): queries times 1 + coef * ln(floor((p + 1) / every) + 1), p the position
//   rotation of the first rot_dim elements of every head ("half-split" pairing, qk_prepare.cuh);
//       elements from rot_dim on pass through
//   queries go to q_out [n, Hq*D]; keys to k_cache[page, slot, key head, :D]; values to
//       v_cache[page, slot, value head, :DV].  v_off < 0: the values ARE the keys as projected (before
//       norm and rotation; Hv == Hk and DV == D then).
//
// Key size D and value size DV are independent, and so are the numbers of key and value heads.  All
// arithmetic is 32-bit (sum of squares, logarithm, angles, cosines, sines).
#include "common.cuh"
#include "qk_prepare.cuh"

namespace {
constexpr int THREADS = 128;
constexpr int ELEMS_PER_BLOCK = 4 * THREADS;

struct PrepareParams {
  const void* proj; long long row_stride; int q_off, k_off, v_off;
  void* q_out;
  const int* positions; const int* token_entry; const int* block_table; int table_width;
  const float* inv_freq; int rot_dim;
  const void* q_norm_w; const void* k_norm_w; float eps;
  float temp_coef; int temp_every;
  void* k_cache; void* v_cache;
  int n_q_heads, n_k_heads, n_v_heads, key_dim, value_dim, page_size, num_pages;
  int* status;
};

// One element of a vector of heads of `dim` elements: the common factor (norm, temperature), the norm's weight,
// and for the first rot_dim elements of a head the rotation with its partner (cosines and sines of the token's
// position come from shared memory: trig[j] = cos, trig[half + j] = sin).
template <typename T, typename TW>
__device__ __forceinline__ float prepare_element(const T* __restrict__ src, int i, int dim, const TW* __restrict__ w,
                                                 float factor, const float* trig, int rot_dim) {
  const int head = i / dim, d = i - head * dim;
  float v = to_f32(src[i]) * factor;
  if (w != nullptr) v *= to_f32(w[i]);
  if (d < rot_dim) {
    const int half = rot_dim >> 1;
    const int j = d < half ? d : d - half;
    const int ip = d < half ? i + half : i - half;          // the partner of the pair
    float u = to_f32(src[ip]) * factor;
    if (w != nullptr) u *= to_f32(w[ip]);
    float first, second;
    if (d < half) qk_rotate_pair(v, u, trig[j], trig[half + j], &first, &second);
    else qk_rotate_pair(u, v, trig[j], trig[half + j], &first, &second);
    v = d < half ? first : second;
  }
  return v;
}

template <typename T>
__device__ __forceinline__ float sum_of_squares(const T* __restrict__ src, int n, float* scratch) {
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += THREADS) {
    const float v = to_f32(src[i]);
    ss += v * v;
  }
  return block_sum(ss, scratch);
}

// grid = (tokens, parts): a block handles ELEMS_PER_BLOCK consecutive elements of the token's [queries | keys |
// values]; every block of a token forms the token's cosines and sines and (for whole-projection norms) the sums of
// squares itself, which is a few thousand elements read from the L2.
template <typename T, typename TW>
__global__ void __launch_bounds__(THREADS) attn_prepare_kernel(const PrepareParams p) {
  extern __shared__ float trig[];                            // [rot_dim / 2] cosines, [rot_dim / 2] sines
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int pos = p.positions[n];
  const T* row = (const T*)p.proj + (size_t)n * p.row_stride;
  const int D = p.key_dim, DV = p.value_dim;
  const bool writes = p.k_cache != nullptr;
  const int nq = p.n_q_heads * D, nk = writes ? p.n_k_heads * D : 0, nv = writes ? p.n_v_heads * DV : 0;
  const int first = blockIdx.y * ELEMS_PER_BLOCK, last = min(first + ELEMS_PER_BLOCK, nq + nk + nv);
  const int half = p.rot_dim >> 1;
  for (int j = threadIdx.x; j < half; j += THREADS) qk_rotation(pos, p.inv_freq[j], &trig[half + j], &trig[j]);

  float q_factor = 1.f, k_factor = 1.f;
  if (p.q_norm_w != nullptr && first < nq) q_factor = qk_norm_factor(sum_of_squares(row + p.q_off, nq, scratch), nq, p.eps);
  if (p.k_norm_w != nullptr && last > nq && first < nq + nk)
    k_factor = qk_norm_factor(sum_of_squares(row + p.k_off, nk, scratch), nk, p.eps);
  if (p.temp_every > 0) q_factor *= 1.f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.f);
  __syncthreads();                                           // the cosines and sines are there

  size_t slot = 0;
  bool have_page = false;
  if (writes && last > nq) {
    const int entry = p.token_entry[n];
    const int page_idx = pos / p.page_size;
    const int page = (page_idx < p.table_width) ? p.block_table[(size_t)entry * p.table_width + page_idx] : -1;
    if (page < 0 || page >= p.num_pages) {
      if (threadIdx.x == 0) atomicOr(p.status, JV_STATUS_BAD_PAGE);
    } else {
      have_page = true;
      slot = (size_t)page * p.page_size + (pos - page_idx * p.page_size);
    }
  }
  T* q_dst = (T*)p.q_out + (size_t)n * nq;
  T* k_dst = (T*)p.k_cache + slot * nk;
  T* v_dst = (T*)p.v_cache + slot * nv;
  const T* v_src = row + (p.v_off >= 0 ? p.v_off : p.k_off);    // the values, or the keys as projected
  for (int idx = first + threadIdx.x; idx < last; idx += THREADS) {
    if (idx < nq) {
      q_dst[idx] = from_f32<T>(prepare_element<T, TW>(row + p.q_off, idx, D, (const TW*)p.q_norm_w, q_factor, trig, p.rot_dim));
    } else if (!have_page) {
      continue;
    } else if (idx < nq + nk) {
      const int i = idx - nq;
      k_dst[i] = from_f32<T>(prepare_element<T, TW>(row + p.k_off, i, D, (const TW*)p.k_norm_w, k_factor, trig, p.rot_dim));
    } else {
      const int i = idx - nq - nk;
      v_dst[i] = v_src[i];
    }
  }
}
}  // namespace

// proj: [n, row_stride] of `dtype`; q_out: [n, n_q_heads*key_dim] of `dtype`; norm weights of `w_dtype`
// ([n_q_heads*key_dim], [n_k_heads*key_dim]) or null; inv_freq: [rot_dim/2] float or null (rot_dim 0);
// temp_every 0: no query temperature; k_cache [num_pages, page_size, n_k_heads, key_dim], v_cache
// [num_pages, page_size, n_v_heads, value_dim] of `dtype`, both null: queries only.
JV_EXPORT int jv_attn_prepare(const void* proj, int dtype, long long row_stride, int q_off, int k_off, int v_off,
                              void* q_out, const int* positions, const int* token_entry, const int* block_table,
                              int table_width, const float* inv_freq, int rot_dim, const void* q_norm_w,
                              const void* k_norm_w, int w_dtype, float eps, float temp_coef, int temp_every,
                              void* k_cache, void* v_cache, int n, int n_q_heads, int n_k_heads, int n_v_heads,
                              int key_dim, int value_dim, int page_size, int num_pages, int* status,
                              cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (rot_dim < 0 || rot_dim > key_dim || (rot_dim & 1) || (rot_dim > 0 && inv_freq == nullptr) || key_dim < 1 ||
      value_dim < 1 || page_size < 1)
    return JV_ERR_UNSUPPORTED;
  if (k_cache != nullptr && v_off < 0 && (n_v_heads != n_k_heads || value_dim != key_dim)) return JV_ERR_UNSUPPORTED;
  PrepareParams p;
  p.proj = proj; p.row_stride = row_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.q_out = q_out;
  p.positions = positions; p.token_entry = token_entry; p.block_table = block_table; p.table_width = table_width;
  p.inv_freq = inv_freq; p.rot_dim = rot_dim; p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.eps = eps;
  p.temp_coef = temp_coef; p.temp_every = temp_every; p.k_cache = k_cache; p.v_cache = v_cache;
  p.n_q_heads = n_q_heads; p.n_k_heads = n_k_heads; p.n_v_heads = n_v_heads; p.key_dim = key_dim;
  p.value_dim = value_dim; p.page_size = page_size; p.num_pages = num_pages; p.status = status;
  const int total = n_q_heads * key_dim + (k_cache != nullptr ? n_k_heads * key_dim + n_v_heads * value_dim : 0);
  const dim3 grid(n, (total + ELEMS_PER_BLOCK - 1) / ELEMS_PER_BLOCK);
  const size_t smem = sizeof(float) * (rot_dim > 0 ? rot_dim : 1);
  JV_DISPATCH_DTYPE(dtype, T, {
    if (w_dtype == 0) return jv_launch(attn_prepare_kernel<T, float>, grid, dim3(THREADS), smem, stream, p);
    if (w_dtype == 1) return jv_launch(attn_prepare_kernel<T, __nv_bfloat16>, grid, dim3(THREADS), smem, stream, p);
  });
  return JV_ERR_UNSUPPORTED;
}
