// Shared helpers for the sm_100a kernels: element types, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SHRIKE_API extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
enum : int { SHRIKE_F32 = 0, SHRIKE_BF16 = 1, SHRIKE_NONE = -1 };

// Status codes returned by every launcher (0 = launched).
enum : int { SHRIKE_OK = 0, SHRIKE_BAD_ARGUMENT = -1 };

static inline int shrike_launch_status() {
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? SHRIKE_OK : static_cast<int>(err);
}

// What launchers need to know of the current device (grids and shared-memory budgets follow
// from it), asked once per device; the figures of a B200 stand in if the query fails.
struct ShrikeDevice {
  int sm_count = 0;
  int max_smem = 0;   // most dynamic shared memory a CTA may ask for
};
static inline const ShrikeDevice& shrike_device() {
  static ShrikeDevice facts[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
  ShrikeDevice& f = facts[device];
  if (f.sm_count == 0) {
    int sms = 0, smem = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
    if (cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess || smem <= 0)
      smem = 227 * 1024;
    f.max_smem = smem;
    f.sm_count = sms;
  }
  return f;
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Four consecutive elements as float32, with one 16-byte (float32) or 8-byte (bfloat16) access.
template <typename TD> __device__ __forceinline__ void load4(const TD* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
template <typename TO> __device__ __forceinline__ void store4(TO* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const unsigned*>(&lo);
  t.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}

// Programmatic dependent launch.  Every kernel of this package is launched so that it may
// start while the kernel before it on the stream is still running (its launch latency and
// set-up are hidden that way), and every kernel begins with
//   let_dependents_start();   the kernel after this one may start now
//   wait_for_previous();      block until the kernel before this one has finished and its
//                             writes are visible
// before it reads or writes any memory that another kernel touches.  Only work on memory
// that no kernel writes (weights) may come before wait_for_previous().
__device__ __forceinline__ void let_dependents_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_previous() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launches `kernel` as a programmatic dependent of the work before it on `stream`.
template <typename... KernelArgs, typename... Args>
static inline cudaError_t launch_dependent(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// The same for a kernel whose CTAs form clusters of `cluster_x` along x (gridDim.x a multiple of it).
template <typename... KernelArgs, typename... Args>
static inline cudaError_t launch_dependent_clusters(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                                    cudaStream_t stream, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  attributes[1].id = cudaLaunchAttributeClusterDimension;
  attributes[1].val.clusterDim.x = cluster_x;
  attributes[1].val.clusterDim.y = 1;
  attributes[1].val.clusterDim.z = 1;
  config.attrs = attributes;
  config.numAttrs = 2;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// silu(g) * u, silu(g) = g / (1 + exp(-g)), with one rounding of the product.  bfloat16 results
// keep 8 bits of mantissa, so that path may use the hardware exponential and reciprocal
// (relative error about 2^-22); the float32 path uses the exact functions.  Shared by the
// activation kernel and the tensor-core product's activation epilogue: both give the same bits.
template <typename T> __device__ __forceinline__ float silu_times(float g, float u);
template <> __device__ __forceinline__ float silu_times<float>(float g, float u) {
  return __fmul_rn(g / (1.0f + expf(-g)), u);
}
template <> __device__ __forceinline__ float silu_times<__nv_bfloat16>(float g, float u) {
  return __fmul_rn(__fdividef(g, 1.0f + __expf(-g)), u);
}

// gelu_tanh(g) * u, gelu_tanh(g) = 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))), with one rounding
// of the product.  As with SiLU, the bfloat16 path may use the hardware exponential
// (tanh(z) = 1 - 2 / (exp(2 z) + 1)); the float32 path uses tanhf.
template <typename T> __device__ __forceinline__ float gelu_tanh_times(float g, float u);
template <> __device__ __forceinline__ float gelu_tanh_times<float>(float g, float u) {
  const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  return __fmul_rn(0.5f * g * (1.0f + tanhf(z)), u);
}
template <> __device__ __forceinline__ float gelu_tanh_times<__nv_bfloat16>(float g, float u) {
  const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  const float t = 1.0f - __fdividef(2.0f, __expf(2.0f * z) + 1.0f);
  return __fmul_rn(0.5f * g * (1.0f + t), u);
}

// The clamped gate: g <- min(g, limit), u <- clamp(u, -limit, limit), then g sigmoid(1.702 g) (u + 1), with one
// rounding of the last product; the exponential as in silu_times.
template <typename T> __device__ __forceinline__ float clamped_swish_times(float g, float u, float limit);
template <> __device__ __forceinline__ float clamped_swish_times<float>(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return __fmul_rn(g / (1.0f + expf(-1.702f * g)), u + 1.0f);
}
template <> __device__ __forceinline__ float clamped_swish_times<__nv_bfloat16>(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return __fmul_rn(__fdividef(g, 1.0f + __expf(-1.702f * g)), u + 1.0f);
}

// Activation codes of the gated feed-forward, shared with the Python side.  `limit` serves the clamped gate alone.
enum : int { SHRIKE_ACT_SILU = 0, SHRIKE_ACT_GELU_TANH = 1, SHRIKE_ACT_CLAMPED_SWISH = 2 };
__host__ __device__ __forceinline__ bool known_activation(int act) { return act >= SHRIKE_ACT_SILU && act <= SHRIKE_ACT_CLAMPED_SWISH; }
template <typename T> __device__ __forceinline__ float act_times(int act, float g, float u, float limit = 0.f) {
  if (act == SHRIKE_ACT_CLAMPED_SWISH) return clamped_swish_times<T>(g, u, limit);
  return act == SHRIKE_ACT_GELU_TANH ? gelu_tanh_times<T>(g, u) : silu_times<T>(g, u);
}

// The first key a query at position `last` sees.  span > 0: the `span` latest keys (a sliding window);
// span < 0: positions are cut into runs of -span counted from position 0, and a query sees its own run only;
// span == 0: every key.  Never decreases as `last` grows, so a tile's first row gives the tile's first key.
__host__ __device__ __forceinline__ int first_visible_key(int last, int span) {
  if (span > 0) return last - span + 1 > 0 ? last - span + 1 : 0;
  if (span < 0) return last > 0 ? (last / -span) * -span : 0;
  return 0;
}

// base[0] + base[stride] + ... over `partials` slices (the stack a K-split product leaves),
// added in ascending order.  Up to 16 loads are issued together before the first addition,
// so the sum costs one memory latency, not one per slice.
__device__ __forceinline__ float sum_partials(const float* base, long long stride, int partials) {
  if (partials == 1) return base[0];
  float held[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) held[i] = (i == 0 || i < partials) ? base[i * stride] : 0.f;
  float sum = held[0];
#pragma unroll
  for (int i = 1; i < 16; ++i)
    if (i < partials) sum = __fadd_rn(sum, held[i]);
  for (int i = 16; i < partials; ++i) sum = __fadd_rn(sum, base[i * stride]);
  return sum;
}

// The same for four consecutive elements with 16-byte loads: v = base[0..3] + base[stride + 0..3] + ...,
// up to eight slices in flight before the first addition, added in ascending order.
__device__ __forceinline__ void sum_partials4(const float* base, long long stride, int partials, float (&v)[4]) {
  load4<float>(base, v);
  for (int first = 1; first < partials; first += 7) {
    float more[7][4];
#pragma unroll
    for (int q = 0; q < 7; ++q)
      if (first + q < partials) load4<float>(base + (first + q) * stride, more[q]);
#pragma unroll
    for (int q = 0; q < 7; ++q)
      if (first + q < partials) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = __fadd_rn(v[e], more[q][e]);
      }
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order
// of additions depends only on the block size, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    float w = lane < warps ? scratch[lane] : 0.f;
    w = warp_sum(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    float w = lane < warps ? scratch[lane] : -INFINITY;
    w = warp_max(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
