// seq_common.cuh -- shared helpers of libb200seq (dense linear layers + sequence operators, sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/b200seq.h"

namespace b200seq {

void count_launch(int n = 1);
int fail(int code, const char* fmt, ...);
int cuda_status(cudaError_t e, const char* what);
int* error_flag_dev();   // device int: bit 0 = KV position outside the block table, bit 1 = bounded wait ran out

#define SEQ_LAUNCH_CHECK(what)                         \
    do {                                               \
        cudaError_t e_ = cudaGetLastError();           \
        if (e_ != cudaSuccess) return cuda_status(e_, what); \
        count_launch();                                \
    } while (0)

__device__ __forceinline__ void store_act(void* out, int dtype, int64_t idx, float v) {
    if (dtype == B200SEQ_F32) reinterpret_cast<float*>(out)[idx] = v;
    else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// sum over the block; every thread gets the result.  red: >= 33 floats of shared memory.  Fixed order: deterministic.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();   // red may still be read from the previous call
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float sigmoidf_acc(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_acc(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_acc(float x) { return x > 20.f ? x : log1pf(expf(x)); }

}  // namespace b200seq
