// seq_attn.cu -- attention of a flat mixed batch (prompt portions beside single decoded tokens) over a paged f32 KV pool.
//   prep  : per-head unit-RMS q and k (no weight), k and v rows stored at the token's page slot.
//   attend: one block per (token, query head); the visible keys are the token's own chunk and / or window, read through the
//           entry's block table; scores, soft-max and the weighted sum in f32; optional per-head sigmoid gate on the output.
// A block's result depends on the token's position and on its sequence's pages only, never on the rest of the batch.
#include "seq_common.cuh"

namespace b200seq {

__device__ __forceinline__ int64_t kv_row(const b200seq_step& st, int e, int pos, int* err) {
    const int b = pos / st.block_size;
    if (b >= st.max_blocks || pos < 0) {
        atomicOr(err, 1);
        return -1;
    }
    return (int64_t)st.block_table[(int64_t)e * st.max_blocks + b] * st.block_size + pos % st.block_size;
}

// grid (T), one warp per head unit: H query heads, G key heads, G value heads
__global__ void attn_prep_kernel(float* __restrict__ qkvg, int64_t ld, b200seq_step st, float* __restrict__ kpool, float* __restrict__ vpool, int H, int G,
                                 int D, int V, float qk_eps, int* err) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int e = st.tok_ent[t];
    const int64_t row = kv_row(st, e, st.tok_pos[t], err);
    float* base = qkvg + (int64_t)t * ld;
    for (int u = wid; u < H + 2 * G; u += nw) {
        if (u < H + G) {   // q or k head: normalise
            float* p = base + (int64_t)u * D;   // q heads then k heads are contiguous
            float rinv = 1.f;
            if (qk_eps >= 0.f) {
                float ss = 0.f;
                for (int d = lane; d < D; d += 32) ss = fmaf(p[d], p[d], ss);
                ss = warp_sum(ss);
                rinv = 1.0f / sqrtf(ss / (float)D + qk_eps);
            }
            if (u < H) {
                for (int d = lane; d < D; d += 32) p[d] *= rinv;
            } else if (row >= 0) {
                float* dst = kpool + (row * G + (u - H)) * D;
                for (int d = lane; d < D; d += 32) dst[d] = p[d] * rinv;
            }
        } else if (row >= 0) {
            const int g = u - H - G;
            const float* p = base + (int64_t)(H + G) * D + (int64_t)g * V;
            float* dst = vpool + (row * G + g) * V;
            for (int d = lane; d < V; d += 32) dst[d] = p[d];
        }
    }
}

constexpr int ATT_WARPS = 4;
constexpr int ATT_VR = 8;   // value elements per lane: V <= 256
// dynamic shared memory: q[D] | per warp: m, l, acc[V]
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_kernel(const float* __restrict__ qkvg, int64_t ld, b200seq_step st, const float* __restrict__ kpool,
                                                              const float* __restrict__ vpool, int H, int G, int D, int V, float scale, int chunk,
                                                              int window, int gated, void* __restrict__ out, int out_dtype, int* err) {
    extern __shared__ float sm[];
    float* qs = sm;
    float* wm = sm + D;                 // [ATT_WARPS]
    float* wl = wm + ATT_WARPS;         // [ATT_WARPS]
    float* wacc = wl + ATT_WARPS;       // [ATT_WARPS][V]
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int e = st.tok_ent[t], pos = st.tok_pos[t];
    const int g = h / (H / G);
    const float* qp = qkvg + (int64_t)t * ld + (int64_t)h * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qp[d];
    __syncthreads();
    int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
    if (window > 0) lo = max(lo, pos - window + 1);
    const int32_t* bt = st.block_table + (int64_t)e * st.max_blocks;
    const int bs = st.block_size;
    if (pos / bs >= st.max_blocks) {
        if (threadIdx.x == 0) atomicOr(err, 1);
        return;
    }
    float m = -INFINITY, l = 0.f, acc[ATT_VR];
#pragma unroll
    for (int i = 0; i < ATT_VR; ++i) acc[i] = 0.f;
    const bool d4 = (D & 3) == 0;
    for (int base = lo + wid * 32; base <= pos; base += ATT_WARPS * 32) {
        const int kp = base + lane;
        float s = -INFINITY;
        if (kp <= pos) {
            const int64_t row = (int64_t)bt[kp / bs] * bs + kp % bs;
            const float* kr = kpool + (row * G + g) * D;
            float a = 0.f;
            if (d4) {
                for (int d = 0; d < D; d += 4) {
                    const float4 kv = *reinterpret_cast<const float4*>(kr + d);
                    a = fmaf(qs[d], kv.x, a), a = fmaf(qs[d + 1], kv.y, a), a = fmaf(qs[d + 2], kv.z, a), a = fmaf(qs[d + 3], kv.w, a);
                }
            } else {
                for (int d = 0; d < D; ++d) a = fmaf(qs[d], kr[d], a);
            }
            s = a * scale;
        }
        const float mn = fmaxf(m, warp_max(s));
        const float corr = expf(m - mn);   // m = -inf on the first tile: exp(-inf) = 0
        const float p = kp <= pos ? expf(s - mn) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < ATT_VR; ++i) acc[i] *= corr;
        m = mn;
        const int nk = min(32, pos - base + 1);
        for (int j = 0; j < nk; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const int kj = base + j;
            const int64_t row = (int64_t)bt[kj / bs] * bs + kj % bs;
            const float* vr = vpool + (row * G + g) * V;
#pragma unroll
            for (int i = 0; i < ATT_VR; ++i) {
                const int d = lane + 32 * i;
                if (d < V) acc[i] = fmaf(pj, vr[d], acc[i]);
            }
        }
    }
    if (lane == 0) wm[wid] = m, wl[wid] = l;
#pragma unroll
    for (int i = 0; i < ATT_VR; ++i) {
        const int d = lane + 32 * i;
        if (d < V) wacc[wid * V + d] = acc[i];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, wm[w]);
    float L = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) L += wm[w] == -INFINITY ? 0.f : wl[w] * expf(wm[w] - M);
    float gate = 1.f;
    if (gated) gate = sigmoidf_acc(qkvg[(int64_t)t * ld + (int64_t)(H + G) * D + (int64_t)G * V + h]);
    for (int d = threadIdx.x; d < V; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w)
            if (wm[w] != -INFINITY) o = fmaf(wacc[w * V + d], expf(wm[w] - M), o);
        store_act(out, out_dtype, (int64_t)t * H * V + (int64_t)h * V + d, o / L * gate);
    }
}

}  // namespace b200seq

using namespace b200seq;

extern "C" {

int b200seq_attn_prep(float* qkvg, int64_t ld, const b200seq_step* st, float* kpool, float* vpool, int H, int G, int D, int V, float qk_eps, void* stream) {
    if (!qkvg || !st || !kpool || !vpool || H < 1 || G < 1 || H % G || D < 1 || V < 1) return fail(B200SEQ_ERR_INVALID_ARG, "attn_prep: bad arguments");
    if (st->T == 0) return 0;
    attn_prep_kernel<<<st->T, 256, 0, (cudaStream_t)stream>>>(qkvg, ld, *st, kpool, vpool, H, G, D, V, qk_eps, error_flag_dev());
    SEQ_LAUNCH_CHECK("attn_prep");
    return 0;
}

int b200seq_attn(const float* qkvg, int64_t ld, const b200seq_step* st, const float* kpool, const float* vpool, int H, int G, int D, int V, float scale,
                 int chunk, int window, int gated, void* out, int out_dtype, void* stream) {
    if (!qkvg || !st || !kpool || !vpool || !out || H < 1 || G < 1 || H % G || D < 1 || V < 1 || V > 32 * ATT_VR)
        return fail(B200SEQ_ERR_INVALID_ARG, "attn: bad arguments (value size <= %d)", 32 * ATT_VR);
    if (st->T == 0) return 0;
    const size_t smem = ((size_t)D + 2 * ATT_WARPS + (size_t)ATT_WARPS * V) * sizeof(float);
    if (smem > 48 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "attn: head size too large");
    dim3 grid(st->T, H);
    attn_kernel<<<grid, ATT_WARPS * 32, smem, (cudaStream_t)stream>>>(qkvg, ld, *st, kpool, vpool, H, G, D, V, scale, chunk, window, gated, out, out_dtype,
                                                                      error_flag_dev());
    SEQ_LAUNCH_CHECK("attn");
    return 0;
}

}  // extern "C"
