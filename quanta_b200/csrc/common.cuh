// Shared device helpers for the quanta_b200 kernels (sm_100a).
//
// Conventions used by every kernel file:
//  * entry points are extern "C", take raw device pointers and a cudaStream_t, allocate nothing,
//    and return 0 or a cudaError_t / negative QB_ERR_* code;
//  * activations are float32 or bfloat16, chosen by a dtype code (QB_F32 / QB_BF16);
//  * statistics, softmax, router scores, rotation angles and the residual stream are float32;
//  * a kernel that is handed an index it cannot honour (token id, page id, expert id) records it in
//    the engine's status words and skips the access instead of faulting.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define QB_F32 0
#define QB_BF16 1

#define QB_ERR_BAD_ARG (-1)
#define QB_ERR_UNSUPPORTED (-2)

// status words written by kernels: [0] first error code, [1] detail, [2] kernel id
#define QB_STATUS_BAD_TOKEN 1
#define QB_STATUS_BAD_PAGE 2
#define QB_STATUS_BAD_EXPERT 3
#define QB_STATUS_WAIT_TIMEOUT 4
#define QB_STATUS_SCRATCH_SMALL 5
#define QB_STATUS_SLOT_MISMATCH 6

#define QB_LAUNCH_CHECK()                        \
  do {                                           \
    cudaError_t e__ = cudaGetLastError();        \
    if (e__ != cudaSuccess) return (int)e__;     \
  } while (0)

__device__ __forceinline__ void qb_set_status(int* status, int code, int detail, int kernel_id) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = detail;
    status[2] = kernel_id;
  }
}

template <typename T> __device__ __forceinline__ float qb_to_float(T v);
template <> __device__ __forceinline__ float qb_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float qb_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T qb_from_float(float v);
template <> __device__ __forceinline__ float qb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 qb_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// 8 consecutive elements at a 16-byte (bfloat16) or 32-byte (float32) aligned address, as floats.
template <typename T> struct QbVec8;
template <> struct QbVec8<float> {
  __device__ static __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ static __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct QbVec8<__nv_bfloat16> {
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = u;
  }
};

__device__ __forceinline__ float qb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float qb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed order (thread partials -> warp tree -> warps in index order), so the
// result for a row never depends on what else is in the batch.  `scratch` holds >= 32 floats.
__device__ __forceinline__ float qb_block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = qb_warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

// Dispatch on a dtype code to a template parameter.
#define QB_DISPATCH_DTYPE(code, T, ...)                                  \
  do {                                                                   \
    if ((code) == QB_F32) { using T = float; __VA_ARGS__; }              \
    else if ((code) == QB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return QB_ERR_BAD_ARG;                                          \
  } while (0)
