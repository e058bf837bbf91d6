// Kernels for layers that norm a branch's OUTPUT (x += norm(branch(x))) and for mixers that
// prepare queries, keys and latents from one fused projection.
//
//   norm_rows      resid += norm(branch) and the sum cast to the activation type, or
//                  out = norm(resid[rows]) for a few gathered rows; RMS or layer norm, bias optional
//   qk_norm_store  queries and keys of a fused q|k projection: RMS over the whole projection (all
//                  heads at once), a position-dependent query temperature, keys into the key pages
//                  and the keys as projected into the value pages
//   latent_store   queries, latent and gate of a fused q|latent|gate projection: queries cast,
//                  the latent RMS-normed into its (one-plane) pages, the gate through a sigmoid
//   head_scale     x[token, head, :] *= gate[token, head]
//
// Statistics, temperature, sigmoid and the residual sum are float32; a result is rounded once, when
// it is stored in the activation type.  Inputs that a K-split product left as a stack of partial
// sums are added in ascending order first.
#include "common.cuh"

namespace branch {

constexpr int MAX_PER_THREAD = 8;

template <typename T> __device__ __forceinline__ float load_sum(const T* base, long long stride, int partials);
template <> __device__ __forceinline__ float load_sum<float>(const float* base, long long stride, int partials) {
  return sum_partials(base, stride, partials);
}
template <> __device__ __forceinline__ float load_sum<__nv_bfloat16>(const __nv_bfloat16* base, long long stride, int partials) {
  float sum = to_float(base[0]);
  for (int i = 1; i < partials; ++i) sum = __fadd_rn(sum, to_float(base[i * stride]));
  return sum;
}

// One block per row; a thread holds elements threadIdx.x + i * blockDim.x in registers between the
// statistics and the scaling, so a row is read once.
//   rows == nullptr: y = norm(sum of the branch's partials); resid[row] += y; out[row] = resid[row]
//                    (out may be null).  branch == nullptr: out[row] = resid[row] only.
//   rows != nullptr: out[r] = norm(resid[rows[r]]); nothing else is written.
// norm(v) = (v - mean) / sqrt(var + eps) * w + b with var the mean squared deviation (layer_norm), or
// v / sqrt(mean(v^2) + eps) * w (+ b).
template <typename TD, typename TO>
__global__ void __launch_bounds__(1024, 1)
norm_rows_kernel(float* __restrict__ resid, const TD* __restrict__ branch, int partials, long long partial_stride,
                 const int* __restrict__ rows, const float* __restrict__ weight, const float* __restrict__ bias,
                 float eps, int layer_norm, TO* __restrict__ out, int width) {
  __shared__ float scratch[33];
  let_dependents_start();
  wait_for_previous();
  const int out_row = blockIdx.x;
  const int row = rows != nullptr ? rows[out_row] : out_row;
  float* x = resid + static_cast<size_t>(row) * width;
  TO* y = out != nullptr ? out + static_cast<size_t>(out_row) * width : nullptr;
  if (rows == nullptr && branch == nullptr) {
    if (y != nullptr)
      for (int i = threadIdx.x; i < width; i += blockDim.x) y[i] = from_float<TO>(x[i]);
    return;
  }
  const TD* d = branch != nullptr ? branch + static_cast<size_t>(row) * width : nullptr;
  float held[MAX_PER_THREAD];
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < MAX_PER_THREAD; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    held[it] = 0.f;
    if (i < width) {
      held[it] = rows != nullptr ? x[i] : load_sum<TD>(d + i, partial_stride, partials);
      sum += held[it];
    }
  }
  float mean = 0.f;
  if (layer_norm) mean = block_sum(sum, scratch) / static_cast<float>(width);
  float sum_sq = 0.f;
#pragma unroll
  for (int it = 0; it < MAX_PER_THREAD; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < width) {
      held[it] -= mean;
      sum_sq = fmaf(held[it], held[it], sum_sq);
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / static_cast<float>(width) + eps);
#pragma unroll
  for (int it = 0; it < MAX_PER_THREAD; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < width) {
      float v = __fmul_rn(__fmul_rn(held[it], inv), weight[i]);
      if (bias != nullptr) v = __fadd_rn(v, bias[i]);
      if (rows == nullptr) {
        v = __fadd_rn(x[i], v);
        x[i] = v;
      }
      if (y != nullptr) y[i] = from_float<TO>(v);
    }
  }
}

// ------------------------------------------------------------ queries and keys of a q|k projection
// One block per token.  qk [P][n][H * D + G * D] float32.  The keys as projected (before their norm)
// are the values.  Heads are stored `padded` (>= D) elements apart, the padding zeroed, so that an
// attention kernel built for the next served head size can read them.
template <typename T>
__global__ void qk_norm_store_kernel(const float* __restrict__ qk, int partials, long long partial_stride,
                                     const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                                     const int* __restrict__ positions, float temp_coef, int temp_every,
                                     T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     const int* __restrict__ slots, int num_heads, int num_kv_heads, int dim, int padded,
                                     long long num_slots) {
  extern __shared__ float row_shared[];   // the token's q and k elements
  __shared__ float scratch[33];
  let_dependents_start();
  const int token = blockIdx.x;
  const int q_width = num_heads * dim, k_width = num_kv_heads * dim;
  long long slot = -1;
  if (k_cache != nullptr) {
    slot = slots[token];
    if (slot < 0 || slot >= num_slots) slot = -1;   // never store outside the pool
  }
  float temperature = 1.0f;
  if (temp_coef != 0.f && temp_every > 0) {
    const int p = positions[token];
    temperature = 1.0f + temp_coef * logf(static_cast<float>((p + 1) / temp_every + 1));
  }
  wait_for_previous();
  const float* row = qk + static_cast<size_t>(token) * (q_width + k_width);
  float q_sq = 0.f, k_sq = 0.f;
  for (int i = threadIdx.x; i < q_width + k_width; i += blockDim.x) {
    const float v = sum_partials(row + i, partial_stride, partials);
    row_shared[i] = v;
    if (i < q_width) q_sq = fmaf(v, v, q_sq);
    else k_sq = fmaf(v, v, k_sq);
  }
  float q_gain = temperature, k_gain = 1.0f;
  if (q_weight != nullptr) q_gain = temperature / sqrtf(block_sum(q_sq, scratch) / static_cast<float>(q_width) + eps);
  if (k_weight != nullptr) k_gain = 1.0f / sqrtf(block_sum(k_sq, scratch) / static_cast<float>(k_width) + eps);
  __syncthreads();
  T* q_dst = q_out + static_cast<size_t>(token) * num_heads * padded;
  for (int i = threadIdx.x; i < num_heads * padded; i += blockDim.x) {
    const int head = i / padded, d = i - head * padded;
    float v = 0.f;
    if (d < dim) {
      const int c = head * dim + d;
      v = row_shared[c] * q_gain;
      if (q_weight != nullptr) v *= q_weight[c];
    }
    q_dst[i] = from_float<T>(v);
  }
  if (slot >= 0) {
    T* k_dst = k_cache + static_cast<size_t>(slot) * num_kv_heads * padded;
    T* v_dst = v_cache + static_cast<size_t>(slot) * num_kv_heads * padded;
    for (int i = threadIdx.x; i < num_kv_heads * padded; i += blockDim.x) {
      const int head = i / padded, d = i - head * padded;
      float k = 0.f, v = 0.f;
      if (d < dim) {
        const int c = head * dim + d;
        v = row_shared[q_width + c];
        k = v * k_gain;
        if (k_weight != nullptr) k *= k_weight[c];
      }
      k_dst[i] = from_float<T>(k);
      v_dst[i] = from_float<T>(v);
    }
  }
}

// ------------------------------------------------- queries, latent and gate of a fused projection
// One block per token.  fused [P][n][q_width + rank + gates] float32 (rank or gates may be 0).
// q_out [n][q_width]; the latent, divided by its root mean square and scaled by `latent_weight`, goes to
// latent_cache[slot][padded] (padding zeroed); gate_out [n][gates] float32 = sigmoid.
template <typename T>
__global__ void latent_store_kernel(const float* __restrict__ fused, int partials, long long partial_stride,
                                    const float* __restrict__ latent_weight, float eps, T* __restrict__ q_out,
                                    T* __restrict__ latent_cache, const int* __restrict__ slots,
                                    float* __restrict__ gate_out, int q_width, int rank, int padded, int gates,
                                    long long num_slots) {
  extern __shared__ float row_shared[];   // the token's latent
  __shared__ float scratch[33];
  let_dependents_start();
  const int token = blockIdx.x;
  long long slot = -1;
  if (latent_cache != nullptr && rank > 0) {
    slot = slots[token];
    if (slot < 0 || slot >= num_slots) slot = -1;
  }
  wait_for_previous();
  const float* row = fused + static_cast<size_t>(token) * (q_width + rank + gates);
  for (int i = threadIdx.x; i < q_width; i += blockDim.x)
    q_out[static_cast<size_t>(token) * q_width + i] = from_float<T>(sum_partials(row + i, partial_stride, partials));
  for (int i = threadIdx.x; i < gates; i += blockDim.x) {
    const float g = sum_partials(row + q_width + rank + i, partial_stride, partials);
    gate_out[static_cast<size_t>(token) * gates + i] = 1.0f / (1.0f + expf(-g));
  }
  if (rank > 0) {
    float sq = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
      const float v = sum_partials(row + q_width + i, partial_stride, partials);
      row_shared[i] = v;
      sq = fmaf(v, v, sq);
    }
    const float gain = 1.0f / sqrtf(block_sum(sq, scratch) / static_cast<float>(rank) + eps);
    if (slot >= 0) {
      T* dst = latent_cache + static_cast<size_t>(slot) * padded;
      for (int i = threadIdx.x; i < padded; i += blockDim.x)
        dst[i] = from_float<T>(i < rank ? row_shared[i] * gain * latent_weight[i] : 0.f);
    }
  }
}

template <typename T>
__global__ void head_scale_kernel(T* __restrict__ x, const float* __restrict__ gate, int heads, int dim) {
  let_dependents_start();
  wait_for_previous();
  const int token = blockIdx.x;
  T* row = x + static_cast<size_t>(token) * heads * dim;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x)
    row[i] = from_float<T>(to_float(row[i]) * gate[static_cast<size_t>(token) * heads + i / dim]);
}

template <typename TD, typename TO>
static int launch_norm_rows(float* resid, const void* branch, int partials, long long partial_stride, const int* rows,
                            const float* weight, const float* bias, float eps, int layer_norm, void* out, int n, int width,
                            cudaStream_t stream) {
  int threads = ((width + MAX_PER_THREAD - 1) / MAX_PER_THREAD + 31) / 32 * 32;
  if (n <= 256) threads = (width + 31) / 32 * 32;   // few rows: latency counts, one element per thread where that fits
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  if (static_cast<long long>(threads) * MAX_PER_THREAD < width) return SHRIKE_BAD_ARGUMENT;
  launch_dependent(norm_rows_kernel<TD, TO>, n, threads, 0, stream, resid, static_cast<const TD*>(branch), partials,
                   partial_stride, rows, weight, bias, eps, layer_norm, static_cast<TO*>(out), width);
  return SHRIKE_OK;
}

}  // namespace branch

// resid [*, width] float32.  rows == null: resid += norm(branch) over n rows, `out` (may be null) gets the
// sum in out_dtype; branch == null: only the cast.  rows != null: out[r] = norm(resid[rows[r]]), n = number of rows.
SHRIKE_API int shrike_norm_rows(float* resid, const void* branch, int branch_dtype, int partials, long long partial_stride,
                                const int* rows, const float* weight, const float* bias, float eps, int layer_norm,
                                void* out, int out_dtype, int n, int width, cudaStream_t stream) {
  using namespace branch;
  if (n <= 0) return SHRIKE_OK;
  if (width <= 0 || partials < 1) return SHRIKE_BAD_ARGUMENT;
  if (rows != nullptr && out == nullptr) return SHRIKE_BAD_ARGUMENT;
  if ((rows != nullptr || branch != nullptr) && weight == nullptr) return SHRIKE_BAD_ARGUMENT;
  if (out != nullptr && out_dtype != SHRIKE_F32 && out_dtype != SHRIKE_BF16) return SHRIKE_BAD_ARGUMENT;
  const bool bf16_branch = branch != nullptr && branch_dtype == SHRIKE_BF16;
  if (branch != nullptr && branch_dtype != SHRIKE_F32 && branch_dtype != SHRIKE_BF16) return SHRIKE_BAD_ARGUMENT;
  int status;
#define SHRIKE_NORM_ROWS(TD, TO) \
  status = launch_norm_rows<TD, TO>(resid, branch, partials, partial_stride, rows, weight, bias, eps, layer_norm, out, n, width, stream)
  if (out_dtype == SHRIKE_BF16 && out != nullptr) {
    if (bf16_branch) SHRIKE_NORM_ROWS(__nv_bfloat16, __nv_bfloat16);
    else SHRIKE_NORM_ROWS(float, __nv_bfloat16);
  } else {
    if (bf16_branch) SHRIKE_NORM_ROWS(__nv_bfloat16, float);
    else SHRIKE_NORM_ROWS(float, float);
  }
#undef SHRIKE_NORM_ROWS
  if (status != SHRIKE_OK) return status;
  return shrike_launch_status();
}

SHRIKE_API int shrike_qk_norm_store(const float* qk, int partials, long long partial_stride, const float* q_weight,
                                    const float* k_weight, float eps, const int* positions, float temp_coef,
                                    int temp_every, void* q_out, void* k_cache, void* v_cache, const int* slots,
                                    int dtype, int n, int num_heads, int num_kv_heads, int dim, int padded,
                                    long long num_slots, cudaStream_t stream) {
  using namespace branch;
  if (n <= 0) return SHRIKE_OK;
  if (partials < 1 || num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || padded < dim) return SHRIKE_BAD_ARGUMENT;
  if ((k_cache == nullptr) != (v_cache == nullptr)) return SHRIKE_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * static_cast<size_t>(num_heads + num_kv_heads) * dim;
  if (smem > static_cast<size_t>(shrike_device().max_smem)) return SHRIKE_BAD_ARGUMENT;
#define SHRIKE_QK_CASE(T)                                                                                    \
  do {                                                                                                       \
    if (smem > 48 * 1024) {                                                                                  \
      const cudaError_t err = cudaFuncSetAttribute(qk_norm_store_kernel<T>,                                  \
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
      if (err != cudaSuccess) return static_cast<int>(err);                                                  \
    }                                                                                                        \
    launch_dependent(qk_norm_store_kernel<T>, n, 256, smem, stream, qk, partials, partial_stride, q_weight,  \
                     k_weight, eps, positions, temp_coef, temp_every, static_cast<T*>(q_out),                \
                     static_cast<T*>(k_cache), static_cast<T*>(v_cache), slots, num_heads, num_kv_heads, dim, \
                     padded, num_slots);                                                                     \
  } while (0)
  if (dtype == SHRIKE_F32) SHRIKE_QK_CASE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_QK_CASE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_QK_CASE
  return shrike_launch_status();
}

SHRIKE_API int shrike_latent_store(const float* fused, int partials, long long partial_stride, const float* latent_weight,
                                   float eps, void* q_out, void* latent_cache, const int* slots, float* gate_out,
                                   int dtype, int n, int q_width, int rank, int padded, int gates, long long num_slots,
                                   cudaStream_t stream) {
  using namespace branch;
  if (n <= 0) return SHRIKE_OK;
  if (partials < 1 || q_width <= 0 || rank < 0 || gates < 0 || padded < rank) return SHRIKE_BAD_ARGUMENT;
  if (rank > 0 && (latent_weight == nullptr || latent_cache == nullptr)) return SHRIKE_BAD_ARGUMENT;
  if (gates > 0 && gate_out == nullptr) return SHRIKE_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * static_cast<size_t>(rank);
  if (smem > 48 * 1024) return SHRIKE_BAD_ARGUMENT;
#define SHRIKE_LATENT_CASE(T)                                                                                  \
  launch_dependent(latent_store_kernel<T>, n, 256, smem, stream, fused, partials, partial_stride, latent_weight, \
                   eps, static_cast<T*>(q_out), static_cast<T*>(latent_cache), slots, gate_out, q_width, rank,  \
                   padded, gates, num_slots)
  if (dtype == SHRIKE_F32) SHRIKE_LATENT_CASE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_LATENT_CASE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_LATENT_CASE
  return shrike_launch_status();
}

SHRIKE_API int shrike_head_scale(void* x, const float* gate, int dtype, int n, int heads, int dim, cudaStream_t stream) {
  using namespace branch;
  if (n <= 0) return SHRIKE_OK;
  if (heads <= 0 || dim <= 0) return SHRIKE_BAD_ARGUMENT;
  if (dtype == SHRIKE_F32) launch_dependent(head_scale_kernel<float>, n, 256, 0, stream, static_cast<float*>(x), gate, heads, dim);
  else if (dtype == SHRIKE_BF16)
    launch_dependent(head_scale_kernel<__nv_bfloat16>, n, 256, 0, stream, static_cast<__nv_bfloat16*>(x), gate, heads, dim);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}
