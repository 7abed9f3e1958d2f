// seq_linear.cu -- dense linear layer y[M,N] = x[M,K] . w[N,K]^T with bfloat16 weights and f32 accumulation.
//   rows  : few tokens (decode).  One warp per pair of weight rows streams them once with 16-byte loads; activations come from L1/L2.
//   tiled : any M in exact f32 arithmetic (fma on f32 operands; bf16 weights widen exactly): the 32-bit path and the small-M fallback.
//   tc    : tcgen05 tiles for bf16 activations (seq_linear_tc.cu).
// The k order of every output element is fixed by the kernel alone, never by M or by the row's place in the batch.
#include "seq_common.cuh"

namespace b200seq {

int launch_linear_tc(const void* x_bf16, int64_t ldx, const void* w_bf16, int M, int N, int K, float* y, int64_t ldy, cudaStream_t st);
bool linear_tc_usable(int x_dtype, int64_t ldx, int M, int N, int K, const void* x, const void* w);
int launch_linear_tc_act(const void* x, int64_t ldx, const void* w, int M, int N, int K, const ActParams act, void* out, int out_dtype, int64_t ldo,
                         cudaStream_t st);

template <typename XT>
__device__ __forceinline__ float ld_x(const XT* p);
template <>
__device__ __forceinline__ float ld_x<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float ld_x<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ void bf16x8_to_f32(const uint4 v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

// MB tokens x 2 weight rows per warp.  VEC: K % 8 == 0 and 16-byte aligned rows (x rows too).
// activation epilogue: act[m][.] is written instead of y.  Gated kinds: the weight is a stacked gate|up with alternating rows, a warp's two
// rows are (gate j, up j) and give output j; plain kinds: every row gives its own output.
struct GateEpi {
    void* out;       // null: plain product to y
    int out_dtype;
    int64_t ldo;
    ActParams act;
};

template <typename XT, int MB, bool VEC>
__global__ void __launch_bounds__(256) linear_rows_kernel(const XT* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w, int M, int N, int K,
                                                          float* __restrict__ y, int64_t ldy, int rows_per_warp, const GateEpi ge) {
    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n0 = warp * rows_per_warp;
    if (n0 >= N) return;
    const bool two = rows_per_warp == 2 && n0 + 1 < N;
    const __nv_bfloat16* w0 = w + (int64_t)n0 * K;
    const __nv_bfloat16* w1 = w + (int64_t)(two ? n0 + 1 : n0) * K;
    for (int m0 = 0; m0 < M; m0 += MB) {
        float acc0[MB], acc1[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc0[m] = acc1[m] = 0.f;
        if (VEC) {
#pragma unroll 4
            for (int k = lane * 8; k < K; k += 256) {
                float a[8], b[8];
                bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(w0 + k)), a);
                bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(w1 + k)), b);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    if (m0 + m < M) {
                        float xv[8];
                        const XT* xp = x + (int64_t)(m0 + m) * ldx + k;
                        if (sizeof(XT) == 4) {
                            const float4 p = __ldg(reinterpret_cast<const float4*>(xp)), q = __ldg(reinterpret_cast<const float4*>(xp) + 1);
                            xv[0] = p.x, xv[1] = p.y, xv[2] = p.z, xv[3] = p.w, xv[4] = q.x, xv[5] = q.y, xv[6] = q.z, xv[7] = q.w;
                        } else {
                            bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(xp)), xv);
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            acc0[m] = fmaf(a[i], xv[i], acc0[m]);
                            acc1[m] = fmaf(b[i], xv[i], acc1[m]);
                        }
                    }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                const float a = __bfloat162float(w0[k]), b = __bfloat162float(w1[k]);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    if (m0 + m < M) {
                        const float xv = ld_x<XT>(x + (int64_t)(m0 + m) * ldx + k);
                        acc0[m] = fmaf(a, xv, acc0[m]);
                        acc1[m] = fmaf(b, xv, acc1[m]);
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const float s0 = warp_sum(acc0[m]), s1 = warp_sum(acc1[m]);
            if (lane == 0 && m0 + m < M) {
                if (ge.out) {
                    if (act_is_gated(ge.act.kind)) {
                        store_act(ge.out, ge.out_dtype, (int64_t)(m0 + m) * ge.ldo + (n0 >> 1), act_gated(ge.act, s0, s1));
                    } else {
                        store_act(ge.out, ge.out_dtype, (int64_t)(m0 + m) * ge.ldo + n0, act_plain(ge.act.kind, s0));
                        if (two) store_act(ge.out, ge.out_dtype, (int64_t)(m0 + m) * ge.ldo + n0 + 1, act_plain(ge.act.kind, s1));
                    }
                } else {
                    y[(int64_t)(m0 + m) * ldy + n0] = s0;
                    if (two) y[(int64_t)(m0 + m) * ldy + n0 + 1] = s1;
                }
            }
        }
    }
}

// 64 x 64 output tile, k step 16, 256 threads x (4 x 4) outputs, f32 fma.
constexpr int TM = 64, TN = 64, TK = 16;
template <typename XT>
__global__ void __launch_bounds__(256) linear_tiled_kernel(const XT* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w, int M, int N, int K,
                                                           float* __restrict__ y, int64_t ldy) {
    __shared__ float xs[TK][TM + 4];
    __shared__ float ws[TK][TN + 4];
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx -> n, ty -> m
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread; consecutive threads walk k (contiguous in memory)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            xs[kk][r] = (m0 + r < M && k < K) ? ld_x<XT>(x + (int64_t)(m0 + r) * ldx + k) : 0.f;
            ws[kk][r] = (n0 + r < N && k < K) ? __bfloat162float(w[(int64_t)(n0 + r) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i], b[i] = ws[kk][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[(int64_t)m * ldy + n] = acc[i][j];
        }
    }
}

template <typename XT>
static void launch_rows(const XT* x, int64_t ldx, const __nv_bfloat16* w, int M, int N, int K, float* y, int64_t ldy, cudaStream_t st,
                        const GateEpi ge = GateEpi{nullptr, 0, 0, ActParams{0, 0.f, 0.f, 0.f}}) {
    const bool vec = K % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                     (ldx * (int64_t)sizeof(XT)) % 16 == 0;
    const int rpw = ((ge.out && act_kind_gated(ge.act.kind)) || (N + 15) / 16 >= 4 * 148) ? 2 : 1;   // few rows: one per warp, so that every SM streams weights
    const int warps = (N + rpw - 1) / rpw;
    const int blocks = (warps + 7) / 8;
    if (M <= 1) {
        if (vec) linear_rows_kernel<XT, 1, true><<<blocks, 256, 0, st>>>(x, ldx, w, M, N, K, y, ldy, rpw, ge);
        else linear_rows_kernel<XT, 1, false><<<blocks, 256, 0, st>>>(x, ldx, w, M, N, K, y, ldy, rpw, ge);
    } else if (M <= 2) {
        if (vec) linear_rows_kernel<XT, 2, true><<<blocks, 256, 0, st>>>(x, ldx, w, M, N, K, y, ldy, rpw, ge);
        else linear_rows_kernel<XT, 2, false><<<blocks, 256, 0, st>>>(x, ldx, w, M, N, K, y, ldy, rpw, ge);
    } else {
        if (vec) linear_rows_kernel<XT, 4, true><<<blocks, 256, 0, st>>>(x, ldx, w, M, N, K, y, ldy, rpw, ge);
        else linear_rows_kernel<XT, 4, false><<<blocks, 256, 0, st>>>(x, ldx, w, M, N, K, y, ldy, rpw, ge);
    }
}

}  // namespace b200seq

using namespace b200seq;

extern "C" int b200seq_linear(const void* x, int x_dtype, int64_t ldx, const void* w, int M, int N, int K, float* y, int64_t ldy, int path, void* stream) {
    if (!x || !w || !y || M < 0 || N < 1 || K < 1 || ldx < K || ldy < N) return fail(B200SEQ_ERR_INVALID_ARG, "linear: bad arguments");
    if (x_dtype != B200SEQ_F32 && x_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "linear: activation dtype");
    if (M == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (path == B200SEQ_PATH_AUTO) {
        if (M <= 8) path = B200SEQ_PATH_ROWS;
        else if (M >= 32 && linear_tc_usable(x_dtype, ldx, M, N, K, x, w)) path = B200SEQ_PATH_TC;
        else path = B200SEQ_PATH_TILED;
    }
    if (path == B200SEQ_PATH_TC) {
        if (!linear_tc_usable(x_dtype, ldx, M, N, K, x, w)) return fail(B200SEQ_ERR_UNSUPPORTED, "linear: the tensor-core path needs bf16 activations, K %% 8 == 0 and 16-byte aligned rows");
        return launch_linear_tc(x, ldx, w, M, N, K, y, ldy, st);
    }
    if (path == B200SEQ_PATH_ROWS) {
        if (x_dtype == B200SEQ_F32) launch_rows((const float*)x, ldx, (const __nv_bfloat16*)w, M, N, K, y, ldy, st);
        else launch_rows((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, M, N, K, y, ldy, st);
    } else if (path == B200SEQ_PATH_TILED) {
        dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
        if (x_dtype == B200SEQ_F32) linear_tiled_kernel<<<grid, 256, 0, st>>>((const float*)x, ldx, (const __nv_bfloat16*)w, M, N, K, y, ldy);
        else linear_tiled_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, M, N, K, y, ldy);
    } else {
        return fail(B200SEQ_ERR_INVALID_ARG, "linear: unknown path %d", path);
    }
    SEQ_LAUNCH_CHECK("linear");
    return 0;
}

extern "C" int b200seq_linear_act(const void* x, int x_dtype, int64_t ldx, const void* w, int M, int N, int K, int act, float limit, float alpha, float shift,
                                  void* out, int out_dtype, int64_t ldo, void* stream) {
    if (!x || !w || !out || M < 0 || N < 1 || K < 1 || ldx < K || !act_kind_known(act)) return fail(B200SEQ_ERR_INVALID_ARG, "linear_act: bad arguments");
    const bool gated = act_kind_gated(act);
    if ((gated && (N & 1)) || ldo < (gated ? N / 2 : N)) return fail(B200SEQ_ERR_INVALID_ARG, "linear_act: output shape");
    if (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "linear_act: output dtype");
    if (x_dtype != B200SEQ_F32 && x_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "linear_act: activation dtype");
    if (M == 0) return 0;
    const ActParams ap{act, limit, alpha, shift};
    if (M <= 8) {   // few tokens: the weight-streaming kernel (gated kinds: a warp's two rows are one (gate, up) pair)
        const GateEpi ge{out, out_dtype, ldo, ap};
        if (x_dtype == B200SEQ_F32) launch_rows((const float*)x, ldx, (const __nv_bfloat16*)w, M, N, K, nullptr, 0, (cudaStream_t)stream, ge);
        else launch_rows((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, M, N, K, nullptr, 0, (cudaStream_t)stream, ge);
        SEQ_LAUNCH_CHECK("linear_act rows");
        return 0;
    }
    if (!linear_tc_usable(x_dtype, ldx, M, N, K, x, w)) return fail(B200SEQ_ERR_UNSUPPORTED, "linear_act: more than 8 rows need bf16 activations, K %% 8 == 0 and 16-byte aligned rows");
    return launch_linear_tc_act(x, ldx, w, M, N, K, ap, out, out_dtype, ldo, (cudaStream_t)stream);
}

extern "C" int b200seq_linear_gated(const void* x, int x_dtype, int64_t ldx, const void* w, int M, int F, int K, float limit, float alpha, float up_shift,
                                    void* out, int out_dtype, int64_t ldo, void* stream) {
    return b200seq_linear_act(x, x_dtype, ldx, w, M, 2 * F, K, B200SEQ_ACT_SWISH_CLAMP, limit, alpha, up_shift, out, out_dtype, ldo, stream);
}
