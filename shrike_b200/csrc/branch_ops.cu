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

template <typename T> __device__ __forceinline__ void load_sum4(const T* base, long long stride, int partials, float (&v)[4]);
template <> __device__ __forceinline__ void load_sum4<float>(const float* base, long long stride, int partials, float (&v)[4]) {
  sum_partials4(base, stride, partials, v);
}
// slice after slice: few registers, for the forms that run many rows (which a K-split product never feeds)
template <typename T>
__device__ __forceinline__ void load_sum4_in_turn(const T* base, long long stride, int partials, float (&v)[4]) {
  load4<T>(base, v);
  for (int p = 1; p < partials; ++p) {
    float more[4];
    load4<T>(base + p * stride, more);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = __fadd_rn(v[e], more[e]);
  }
}
template <> __device__ __forceinline__ void load_sum4<__nv_bfloat16>(const __nv_bfloat16* base, long long stride, int partials,
                                                                     float (&v)[4]) {
  load_sum4_in_turn<__nv_bfloat16>(base, stride, partials, v);
}

template <typename T> __device__ __forceinline__ float load_sum(const T* base, long long stride, int partials);
template <> __device__ __forceinline__ float load_sum<float>(const float* base, long long stride, int partials) {
  return sum_partials(base, stride, partials);
}
template <> __device__ __forceinline__ float load_sum<__nv_bfloat16>(const __nv_bfloat16* base, long long stride, int partials) {
  float sum = to_float(base[0]);
  for (int i = 1; i < partials; ++i) sum = __fadd_rn(sum, to_float(base[i * stride]));
  return sum;
}

// One block per row; a thread holds its groups of VEC elements (group threadIdx.x + i * blockDim.x) in
// registers between the statistics and the scaling, so a row is read once; VEC = 4 uses 16-byte accesses.
//   rows == nullptr: y = norm(sum of the branch's partials); resid[row] += y; out[row] = resid[row]
//                    (out may be null).  branch == nullptr: out[row] = resid[row] only.
//   rows != nullptr: out[r] = norm(resid[rows[r]]); nothing else is written.
// norm(v) = (v - mean) / sqrt(var + eps) * w + b with var the mean squared deviation (layer_norm), or
// v / sqrt(mean(v^2) + eps) * w (+ b).
// PT: groups a thread may hold.  PT <= 2 (few rows, decoding: latency counts) reads the norm's weight and bias
// before the wait (no kernel writes them) and has the residual and the branch's slices in flight together, so
// that the row costs one memory round trip; PT = 4 or 8 (many rows: bandwidth counts) reads them where it needs
// them.  PT = 4 (rows of up to 1,024 groups) is built for five blocks of up to 256 threads an SM: with the 64
// registers a block of 1,024 threads may take, four blocks of 224 threads fit and the loads of 41 % of the
// SM's warps are all that is in flight (measured: 3.5 TB/s at rows of 3,584).
template <typename TD, typename TO, int VEC, int PT>
__global__ void __launch_bounds__(PT == 4 ? 256 : 1024, PT == 4 ? 5 : 1)
norm_rows_kernel(float* __restrict__ resid, const TD* __restrict__ branch, int partials, long long partial_stride,
                 const int* __restrict__ rows, const float* __restrict__ weight, const float* __restrict__ bias,
                 float eps, int layer_norm, TO* __restrict__ out, int width) {
  __shared__ float scratch[33];
  constexpr bool EARLY = PT <= 2;
  let_dependents_start();
  const int groups = width / VEC;
  float gain[EARLY ? PT : 1][VEC], shift[EARLY ? PT : 1][VEC];
  if (EARLY && weight != nullptr) {
#pragma unroll
    for (int it = 0; it < (EARLY ? PT : 0); ++it) {
      const int g = threadIdx.x + it * blockDim.x;
      if (g < groups) {
        if (VEC == 4) {
          float w[4], b[4] = {0.f, 0.f, 0.f, 0.f};
          load4<float>(weight + g * 4, w);
          if (bias != nullptr) load4<float>(bias + g * 4, b);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            gain[EARLY ? it : 0][e % VEC] = w[e];
            shift[EARLY ? it : 0][e % VEC] = b[e];
          }
        } else {
          gain[EARLY ? it : 0][0] = weight[g];
          shift[EARLY ? it : 0][0] = bias != nullptr ? bias[g] : 0.f;
        }
      }
    }
  }
  wait_for_previous();
  const int out_row = blockIdx.x;
  const int row = rows != nullptr ? rows[out_row] : out_row;
  float* x = resid + static_cast<size_t>(row) * width;
  TO* y = out != nullptr ? out + static_cast<size_t>(out_row) * width : nullptr;
  if (rows == nullptr && branch == nullptr) {
    if (y != nullptr)
      for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        if (VEC == 4) {
          float v[4];
          load4<float>(x + g * 4, v);
          store4<TO>(y + g * 4, v);
        } else {
          y[g] = from_float<TO>(x[g]);
        }
      }
    return;
  }
  const TD* d = branch != nullptr ? branch + static_cast<size_t>(row) * width : nullptr;
  float held[PT][VEC], before[EARLY ? PT : 1][VEC];
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < PT; ++it) {
    const int g = threadIdx.x + it * blockDim.x;
#pragma unroll
    for (int e = 0; e < VEC; ++e) held[it][e] = 0.f;
    if (g < groups) {
      if (VEC == 4) {
        float v[4];
        if (rows != nullptr) {
          load4<float>(x + g * 4, v);
        } else {
          if (EARLY) {   // the residual's loads go out with the slices'
            float r[4];
            load4<float>(x + g * 4, r);
#pragma unroll
            for (int e = 0; e < 4; ++e) before[EARLY ? it : 0][e % VEC] = r[e];
          }
          // the slices of a K-split product, in ascending order
          if (EARLY) load_sum4<TD>(d + g * 4, partial_stride, partials, v);
          else load_sum4_in_turn<TD>(d + g * 4, partial_stride, partials, v);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) held[it][e % VEC] = v[e];
      } else {
        if (EARLY && rows == nullptr) before[EARLY ? it : 0][0] = x[g];
        held[it][0] = rows != nullptr ? x[g] : load_sum<TD>(d + g, partial_stride, partials);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) sum += held[it][e];
    }
  }
  float mean = 0.f;
  if (layer_norm) mean = block_sum(sum, scratch) / static_cast<float>(width);
  float sum_sq = 0.f;
#pragma unroll
  for (int it = 0; it < PT; ++it) {
    const int g = threadIdx.x + it * blockDim.x;
    if (g < groups) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        held[it][e] -= mean;
        sum_sq = fmaf(held[it][e], held[it][e], sum_sq);
      }
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / static_cast<float>(width) + eps);
#pragma unroll
  for (int it = 0; it < PT; ++it) {
    const int g = threadIdx.x + it * blockDim.x;
    if (g < groups) {
      if (VEC == 4) {
        float w[4], b[4] = {0.f, 0.f, 0.f, 0.f}, r[4];
        if (EARLY) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            w[e] = gain[EARLY ? it : 0][e % VEC];
            b[e] = shift[EARLY ? it : 0][e % VEC];
          }
        } else {
          load4<float>(weight + g * 4, w);
          if (bias != nullptr) load4<float>(bias + g * 4, b);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          r[e] = __fmul_rn(__fmul_rn(held[it][e % VEC], inv), w[e]);
          if (bias != nullptr) r[e] = __fadd_rn(r[e], b[e]);
        }
        if (rows == nullptr) {
          float old[4];
          if (EARLY) {
#pragma unroll
            for (int e = 0; e < 4; ++e) old[e] = before[EARLY ? it : 0][e % VEC];
          } else {
            load4<float>(x + g * 4, old);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) r[e] = __fadd_rn(old[e], r[e]);
          store4<float>(x + g * 4, r);
        }
        if (y != nullptr) store4<TO>(y + g * 4, r);
      } else {
        float v = __fmul_rn(__fmul_rn(held[it][0], inv), EARLY ? gain[EARLY ? it : 0][0] : weight[g]);
        if (bias != nullptr) v = __fadd_rn(v, EARLY ? shift[EARLY ? it : 0][0] : bias[g]);
        if (rows == nullptr) {
          v = __fadd_rn(EARLY ? before[EARLY ? it : 0][0] : x[g], v);
          x[g] = v;
        }
        if (y != nullptr) y[g] = from_float<TO>(v);
      }
    }
  }
}

// ------------------------------------------------------------ queries and keys of a q|k projection
// One block per token.  qk [P][n][H * D + G * D] float32.  The keys as projected (before their norm)
// are the values.  Heads are stored `padded` (>= D) elements apart, the padding zeroed, so that an
// attention kernel built for the next served head size can read them.
template <typename T, int VEC>
__global__ void qk_norm_store_kernel(const float* __restrict__ qk, int partials, long long partial_stride,
                                     const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                                     const int* __restrict__ positions, float temp_coef, int temp_every,
                                     T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     const int* __restrict__ slots, int num_heads, int num_kv_heads, int dim, int padded,
                                     long long num_slots) {
  extern __shared__ __align__(16) float row_shared[];   // the token's q and k elements
  __shared__ float scratch[33];
  let_dependents_start();
  // before the wait: what no kernel writes (the step's positions and slots)
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
  for (int g = threadIdx.x; g < (q_width + k_width) / VEC; g += blockDim.x) {
    const int i = g * VEC;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (VEC == 4) {
      sum_partials4(row + i, partial_stride, partials, v);
      *reinterpret_cast<float4*>(row_shared + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      v[0] = sum_partials(row + i, partial_stride, partials);
      row_shared[i] = v[0];
    }
    float sq = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e) sq = fmaf(v[e], v[e], sq);
    if (i < q_width) q_sq += sq;   // a group never holds elements of both: q_width is a multiple of VEC
    else k_sq += sq;
  }
  float q_gain = temperature, k_gain = 1.0f;
  if (q_weight != nullptr) q_gain = temperature / sqrtf(block_sum(q_sq, scratch) / static_cast<float>(q_width) + eps);
  if (k_weight != nullptr) k_gain = 1.0f / sqrtf(block_sum(k_sq, scratch) / static_cast<float>(k_width) + eps);
  __syncthreads();
  const int per_head = padded / VEC;
  T* q_dst = q_out + static_cast<size_t>(token) * num_heads * padded;
  for (int g = threadIdx.x; g < num_heads * per_head; g += blockDim.x) {
    const int head = g / per_head, d = (g - head * per_head) * VEC;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (d < dim) {   // a group is inside the head or all padding: dim is a multiple of VEC
      const int c = head * dim + d;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        v[e] = row_shared[c + e] * q_gain;
        if (q_weight != nullptr) v[e] *= q_weight[c + e];
      }
    }
    if (VEC == 4) store4<T>(q_dst + head * padded + d, v);
    else q_dst[head * padded + d] = from_float<T>(v[0]);
  }
  if (slot >= 0) {
    T* k_dst = k_cache + static_cast<size_t>(slot) * num_kv_heads * padded;
    T* v_dst = v_cache + static_cast<size_t>(slot) * num_kv_heads * padded;
    for (int g = threadIdx.x; g < num_kv_heads * per_head; g += blockDim.x) {
      const int head = g / per_head, d = (g - head * per_head) * VEC;
      float k[4] = {0.f, 0.f, 0.f, 0.f}, v[4] = {0.f, 0.f, 0.f, 0.f};
      if (d < dim) {
        const int c = head * dim + d;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          v[e] = row_shared[q_width + c + e];
          k[e] = v[e] * k_gain;
          if (k_weight != nullptr) k[e] *= k_weight[c + e];
        }
      }
      if (VEC == 4) {
        store4<T>(k_dst + head * padded + d, k);
        store4<T>(v_dst + head * padded + d, v);
      } else {
        k_dst[head * padded + d] = from_float<T>(k[0]);
        v_dst[head * padded + d] = from_float<T>(v[0]);
      }
    }
  }
}

// ------------------------------------------------- queries, latent and gate of a fused projection
// One block per token.  fused [P][n][row_width] float32, of which the first q_width + rank + gates columns
// are used (rank or gates may be 0; a row may be padded to a width the matrix product likes).
// q_out [n][q_width]; the latent, divided by its root mean square and scaled by `latent_weight`, goes to
// latent_cache[slot][padded] (padding zeroed); gate_out [n][gates] float32 = sigmoid.
template <typename T>
__global__ void latent_store_kernel(const float* __restrict__ fused, int partials, long long partial_stride,
                                    const float* __restrict__ latent_weight, float eps, T* __restrict__ q_out,
                                    T* __restrict__ latent_cache, const int* __restrict__ slots,
                                    float* __restrict__ gate_out, int q_width, int rank, int padded, int gates,
                                    int row_width, long long num_slots, int vec) {
  extern __shared__ __align__(16) float row_shared[];   // the token's latent
  __shared__ float scratch[33];
  let_dependents_start();
  const int token = blockIdx.x;
  long long slot = -1;
  if (latent_cache != nullptr && rank > 0) {
    slot = slots[token];
    if (slot < 0 || slot >= num_slots) slot = -1;
  }
  wait_for_previous();
  const float* row = fused + static_cast<size_t>(token) * row_width;
  if (vec) {   // the queries are the wide part: 16-byte loads, every slice of a K-split product in flight together
    for (int g = threadIdx.x; g < q_width / 4; g += blockDim.x) {
      float v[4];
      sum_partials4(row + g * 4, partial_stride, partials, v);
      store4<T>(q_out + static_cast<size_t>(token) * q_width + g * 4, v);
    }
  } else {
    for (int i = threadIdx.x; i < q_width; i += blockDim.x)
      q_out[static_cast<size_t>(token) * q_width + i] = from_float<T>(sum_partials(row + i, partial_stride, partials));
  }
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

// x [n][heads][dim] in place; a thread takes four elements (dim is a multiple of 4), blockIdx.y the token
template <typename T>
__global__ void head_scale_kernel(T* __restrict__ x, const float* __restrict__ gate, int heads, int dim, int n) {
  let_dependents_start();
  wait_for_previous();
  const int per_row = heads * dim / 4;
  for (int token = blockIdx.y; token < n; token += gridDim.y) {
    T* row = x + static_cast<size_t>(token) * heads * dim;
    const float* g = gate + static_cast<size_t>(token) * heads;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < per_row; i += gridDim.x * blockDim.x) {
      float v[4];
      load4<T>(row + i * 4, v);
      const float scale = g[i * 4 / dim];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] *= scale;
      store4<T>(row + i * 4, v);
    }
  }
}

template <typename TD, typename TO>
static int launch_norm_rows(float* resid, const void* branch, int partials, long long partial_stride, const int* rows,
                            const float* weight, const float* bias, float eps, int layer_norm, void* out, int n, int width,
                            cudaStream_t stream) {
  const uintptr_t addresses = reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(branch) |
                              reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(bias) |
                              reinterpret_cast<uintptr_t>(out);
  const bool vec = width % 4 == 0 && addresses % 16 == 0 && (partials == 1 || partial_stride % 4 == 0);
  const int groups = vec ? width / 4 : width;
  // many rows (prompts): bandwidth counts, small blocks whose threads keep several groups in flight;
  // few rows (decoding): latency counts, one group per thread (two for rows beyond 1024 groups)
  const bool few = n <= 256 && groups <= 2048;
  const bool two = few && groups > 1024;
  int threads = few ? ((two ? (groups + 1) / 2 : groups) + 31) / 32 * 32 : ((groups + 3) / 4 + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  if (static_cast<long long>(threads) * MAX_PER_THREAD < groups) return SHRIKE_BAD_ARGUMENT;
  const bool four = !few && threads <= 256;   // rows of up to 1,024 groups: four groups a thread
#define SHRIKE_NORM_ROWS_LAUNCH(V, P)                                                                              \
  launch_dependent(norm_rows_kernel<TD, TO, V, P>, n, threads, 0, stream, resid, static_cast<const TD*>(branch), partials, \
                   partial_stride, rows, weight, bias, eps, layer_norm, static_cast<TO*>(out), width)
  if (vec) {
    if (two) SHRIKE_NORM_ROWS_LAUNCH(4, 2);
    else if (few) SHRIKE_NORM_ROWS_LAUNCH(4, 1);
    else if (four) SHRIKE_NORM_ROWS_LAUNCH(4, 4);
    else SHRIKE_NORM_ROWS_LAUNCH(4, MAX_PER_THREAD);
  } else {
    if (two) SHRIKE_NORM_ROWS_LAUNCH(1, 2);
    else if (few) SHRIKE_NORM_ROWS_LAUNCH(1, 1);
    else if (four) SHRIKE_NORM_ROWS_LAUNCH(1, 4);
    else SHRIKE_NORM_ROWS_LAUNCH(1, MAX_PER_THREAD);
  }
#undef SHRIKE_NORM_ROWS_LAUNCH
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
  const uintptr_t addresses = reinterpret_cast<uintptr_t>(qk) | reinterpret_cast<uintptr_t>(q_out) |
                              reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache);
  const bool vec = dim % 4 == 0 && padded % 4 == 0 && addresses % 16 == 0 && (partials == 1 || partial_stride % 4 == 0);
  // few tokens (decoding): a thread a group, so that a token's loads are one round trip; many: small blocks
  const int row_groups = (num_heads + num_kv_heads) * dim / (vec ? 4 : 1);
  int threads = n > 256 ? 128 : 256;
  if (n <= 64) threads = row_groups >= 1024 ? 1024 : (row_groups + 31) / 32 * 32 < 128 ? 128 : (row_groups + 31) / 32 * 32;
#define SHRIKE_QK_LAUNCH(T, V)                                                                               \
  do {                                                                                                       \
    if (smem > 48 * 1024) {                                                                                  \
      const cudaError_t err = cudaFuncSetAttribute(qk_norm_store_kernel<T, V>,                               \
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
      if (err != cudaSuccess) return static_cast<int>(err);                                                  \
    }                                                                                                        \
    launch_dependent(qk_norm_store_kernel<T, V>, n, threads, smem, stream, qk, partials, partial_stride,     \
                     q_weight, k_weight, eps, positions, temp_coef, temp_every, static_cast<T*>(q_out),      \
                     static_cast<T*>(k_cache), static_cast<T*>(v_cache), slots, num_heads, num_kv_heads, dim, \
                     padded, num_slots);                                                                     \
  } while (0)
#define SHRIKE_QK_CASE(T) do { if (vec) SHRIKE_QK_LAUNCH(T, 4); else SHRIKE_QK_LAUNCH(T, 1); } while (0)
  if (dtype == SHRIKE_F32) SHRIKE_QK_CASE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_QK_CASE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_QK_LAUNCH
#undef SHRIKE_QK_CASE
  return shrike_launch_status();
}

SHRIKE_API int shrike_latent_store(const float* fused, int partials, long long partial_stride, const float* latent_weight,
                                   float eps, void* q_out, void* latent_cache, const int* slots, float* gate_out,
                                   int dtype, int n, int q_width, int rank, int padded, int gates, int row_width,
                                   long long num_slots, cudaStream_t stream) {
  using namespace branch;
  if (n <= 0) return SHRIKE_OK;
  if (partials < 1 || q_width <= 0 || rank < 0 || gates < 0 || padded < rank || row_width < q_width + rank + gates)
    return SHRIKE_BAD_ARGUMENT;
  if (rank > 0 && latent_weight == nullptr) return SHRIKE_BAD_ARGUMENT;   // without pages the latent is only skipped over
  if (gates > 0 && gate_out == nullptr) return SHRIKE_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * static_cast<size_t>(rank);
  if (smem > 48 * 1024) return SHRIKE_BAD_ARGUMENT;
  const int vec = q_width % 4 == 0 && row_width % 4 == 0 && (partials == 1 || partial_stride % 4 == 0) &&
                  (reinterpret_cast<uintptr_t>(fused) | reinterpret_cast<uintptr_t>(q_out)) % 16 == 0;
#define SHRIKE_LATENT_CASE(T)                                                                                  \
  launch_dependent(latent_store_kernel<T>, n, 256, smem, stream, fused, partials, partial_stride, latent_weight, \
                   eps, static_cast<T*>(q_out), static_cast<T*>(latent_cache), slots, gate_out, q_width, rank,  \
                   padded, gates, row_width, num_slots, vec)
  if (dtype == SHRIKE_F32) SHRIKE_LATENT_CASE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_LATENT_CASE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_LATENT_CASE
  return shrike_launch_status();
}

SHRIKE_API int shrike_head_scale(void* x, const float* gate, int dtype, int n, int heads, int dim, cudaStream_t stream) {
  using namespace branch;
  if (n <= 0) return SHRIKE_OK;
  if (heads <= 0 || dim <= 0 || dim % 4 || reinterpret_cast<uintptr_t>(x) % 16) return SHRIKE_BAD_ARGUMENT;
  const int per_row = heads * dim / 4;
  const dim3 grid(max(1, min(8, (per_row + 255) / 256)), max(1, min(n, 65535)));
  if (dtype == SHRIKE_F32) launch_dependent(head_scale_kernel<float>, grid, 256, 0, stream, static_cast<float*>(x), gate, heads, dim, n);
  else if (dtype == SHRIKE_BF16)
    launch_dependent(head_scale_kernel<__nv_bfloat16>, grid, 256, 0, stream, static_cast<__nv_bfloat16*>(x), gate, heads, dim, n);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}
