// seq_depth.cu -- what lies between two layers of a model whose residual stream is averaged over depth: the residual sum of the layer
// that ended (input + mixer branch + feed-forward branch, both branches read the same input), the learned average over the results
// of all layers so far (which becomes the next layer's input), and the layer norm(s) of that input -- one pass, one block per row,
// all of it in f32.  The statistics of the layer norm are shared by the two norms of a parallel layer (same input, two weights).
#include "seq_common.cuh"

namespace b200seq {

struct DepthArgs {
    const float* hist;       // [n_prev][hist_stride]: X_0 .. X_(n_prev - 1), rows of W
    int64_t hist_stride;
    int n_prev;
    const float* dwa;        // [n_prev + 1] or null
    const float *x_cur, *y1, *y2;
    float *hist_out, *x_out;
    int W;
    float eps;
    const float *w1, *w2;
    const int32_t* rows;
    void *out1, *out2;
    int out_dtype;
};

// dynamic shared memory: W floats (the row) + 40 floats of reduction scratch.  VW = 4: 16-byte accesses.
template <int VW>
__global__ void depth_norm_kernel(const DepthArgs a) {
    extern __shared__ __align__(16) float sm[];
    float* u = sm;
    float* red = sm + a.W;
    const int r = blockIdx.x;
    const int64_t t = a.rows ? a.rows[r] : r;
    const int W = a.W;
    const int64_t base = t * W;
    float part = 0.f;
    for (int i = threadIdx.x * VW; i < W; i += blockDim.x * VW) {
        float x[VW];
        auto ld = [&](const float* p, float* v) {
            if (VW == 4) {
                const float4 q = *reinterpret_cast<const float4*>(p);
                v[0] = q.x, v[1 % VW] = q.y, v[2 % VW] = q.z, v[3 % VW] = q.w;
            } else {
                v[0] = *p;
            }
        };
        auto st = [&](float* p, const float* v) {
            if (VW == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1 % VW], v[2 % VW], v[3 % VW]);
            else *p = v[0];
        };
        ld(a.x_cur + base + i, x);
        if (a.y1) {
            float m[VW];
            ld(a.y1 + base + i, m);
            if (a.y2) {
                float f[VW];
                ld(a.y2 + base + i, f);
#pragma unroll
                for (int e = 0; e < VW; ++e) m[e] += f[e];
            }
#pragma unroll
            for (int e = 0; e < VW; ++e) x[e] += m[e];
            if (a.hist_out) st(a.hist_out + base + i, x);
            if (a.dwa) {
                float acc[VW];
#pragma unroll
                for (int e = 0; e < VW; ++e) acc[e] = 0.f;
                for (int j = 0; j < a.n_prev; ++j) {
                    float h[VW];
                    ld(a.hist + (int64_t)j * a.hist_stride + base + i, h);
                    const float wj = a.dwa[j];
#pragma unroll
                    for (int e = 0; e < VW; ++e) acc[e] = fmaf(wj, h[e], acc[e]);
                }
                const float wl = a.dwa[a.n_prev];
#pragma unroll
                for (int e = 0; e < VW; ++e) x[e] = fmaf(wl, x[e], acc[e]);
            }
            if (a.x_out) st(a.x_out + base + i, x);
        }
#pragma unroll
        for (int e = 0; e < VW; ++e) {
            u[i + e] = x[e];
            part += x[e];
        }
    }
    if (!a.out1 && !a.out2) return;
    const float mean = block_sum(part, red) / (float)W;    // block_sum's barriers also publish u
    float sq = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float d = u[i] - mean;
        sq = fmaf(d, d, sq);
    }
    const float rinv = 1.0f / sqrtf(block_sum(sq, red) / (float)W + a.eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float n = (u[i] - mean) * rinv;
        if (a.out1) store_act(a.out1, a.out_dtype, (int64_t)r * W + i, n * a.w1[i]);
        if (a.out2) store_act(a.out2, a.out_dtype, (int64_t)r * W + i, n * a.w2[i]);
    }
}

}  // namespace b200seq

using namespace b200seq;

extern "C" int b200seq_depth_norm(const float* hist, int64_t hist_stride, int n_prev, const float* dwa, const float* x_cur, const float* y1, const float* y2,
                                  float* hist_out, float* x_out, int W, float eps, const float* w1, const float* w2, const int32_t* rows, int R, void* out1,
                                  void* out2, int out_dtype, void* stream) {
    if (!x_cur || W < 1 || R < 0 || n_prev < 0 || (y2 && !y1) || (dwa && (!y1 || (n_prev > 0 && !hist))) || (out1 && !w1) || (out2 && !w2))
        return fail(B200SEQ_ERR_INVALID_ARG, "depth_norm: bad arguments");
    if (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "depth_norm: output dtype");
    if (R == 0) return 0;
    const size_t smem = ((size_t)W + 40) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "depth_norm: width %d too large", W);
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = W % 4 == 0 && hist_stride % 4 == 0 && al(hist) && al(x_cur) && al(y1) && al(y2) && al(hist_out) && al(x_out);
    const DepthArgs a{hist, hist_stride, n_prev, dwa, x_cur, y1, y2, hist_out, x_out, W, eps, w1, w2, rows, out1, out2, out_dtype};
    const int nt = W >= 4096 ? 512 : (W >= 1024 ? 256 : 128);
    cudaError_t e = cudaSuccess;
    if (vec) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(depth_norm_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) depth_norm_kernel<4><<<R, nt, smem, (cudaStream_t)stream>>>(a);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(depth_norm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) depth_norm_kernel<1><<<R, nt, smem, (cudaStream_t)stream>>>(a);
    }
    if (e != cudaSuccess) return cuda_status(e, "depth_norm attribute");
    SEQ_LAUNCH_CHECK("depth_norm");
    return 0;
}
