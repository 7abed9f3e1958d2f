// seq_ssm.cu -- selective state-space recurrence (scalar decay per head, state N x V per head) over a flat mixed batch.
// One warp per (32 value columns, head, entry); each lane keeps its column of the state (N floats) in registers and walks the
// entry's tokens in order; B, C, the step sizes and the decays of a tile of tokens are staged in shared memory.
// Step sizes, decays and the state are f32; the state is read from / written to the sequence's slot (zero for a new sequence).
#include "seq_common.cuh"

namespace b200seq {

constexpr int SSM_TT = 16;   // tokens per staged tile

template <int NPT>
__global__ void __launch_bounds__(32) ssm_scan_kernel(const float* __restrict__ proj, int64_t ldp, int z0, int dt0, const float* __restrict__ xbc, int64_t ldx,
                                                      const float* __restrict__ A_log, const float* __restrict__ Dp, const float* __restrict__ dt_bias,
                                                      float* __restrict__ state, b200seq_step st, int H, int V, int N, int G, float* __restrict__ out) {
    extern __shared__ float sm[];
    float* Bs = sm;                      // [SSM_TT][N]
    float* Cs = Bs + SSM_TT * N;         // [SSM_TT][N]
    float* dts = Cs + SSM_TT * N;        // [SSM_TT]
    float* dec = dts + SSM_TT;           // [SSM_TT]
    const int lane = threadIdx.x;
    const int v = blockIdx.x * 32 + lane;
    const int h = blockIdx.y, e = blockIdx.z;
    const int s0 = st.ent_start[e], len = st.ent_start[e + 1] - s0;
    const bool fresh = st.ent_pos0[e] == 0;
    const bool live = v < V;
    const int g = h / (H / G);
    const int inner = H * V;
    float* sp = state + (((int64_t)st.ent_slot[e] * H + h) * N) * V + v;
    float S[NPT];
#pragma unroll
    for (int n = 0; n < NPT; ++n) S[n] = (live && !fresh && n < N) ? sp[(int64_t)n * V] : 0.f;
    const float negA = -expf(A_log[h]);
    const float dtb = dt_bias[h], Dh = Dp[h];
    for (int i0 = 0; i0 < len; i0 += SSM_TT) {
        const int nt = min(SSM_TT, len - i0);
        __syncwarp();
        for (int idx = lane; idx < nt * N; idx += 32) {
            const int tt = idx / N, n = idx - tt * N;
            const float* r = xbc + (int64_t)(s0 + i0 + tt) * ldx + inner + (int64_t)g * N + n;
            Bs[tt * N + n] = r[0];
            Cs[tt * N + n] = r[(int64_t)G * N];
        }
        if (lane < nt) {
            const float dt = softplusf_acc(proj[(int64_t)(s0 + i0 + lane) * ldp + dt0 + h] + dtb);
            dts[lane] = dt;
            dec[lane] = expf(negA * dt);
        }
        __syncwarp();
        if (live) {
            for (int tt = 0; tt < nt; ++tt) {
                const int64_t row = s0 + i0 + tt;
                const float x = xbc[row * ldx + (int64_t)h * V + v];
                const float z = proj[row * ldp + z0 + (int64_t)h * V + v];
                const float dA = dec[tt], dtx = dts[tt] * x;
                const float* Bt = Bs + tt * N;
                const float* Ct = Cs + tt * N;
                float y = 0.f;
#pragma unroll
                for (int n = 0; n < NPT; ++n) {
                    if (n < N) {
                        S[n] = fmaf(dA, S[n], dtx * Bt[n]);
                        y = fmaf(S[n], Ct[n], y);
                    }
                }
                y = fmaf(Dh, x, y);
                out[row * inner + (int64_t)h * V + v] = y * siluf_acc(z);
            }
        }
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < NPT; ++n)
            if (n < N) sp[(int64_t)n * V] = S[n];
    }
}

}  // namespace b200seq

using namespace b200seq;

extern "C" int b200seq_ssm_scan(const float* proj, int64_t ldp, int z0, int dt0, const float* xbc, int64_t ldx, const float* A_log, const float* Dp,
                                const float* dt_bias, float* state, const b200seq_step* st, int H, int V, int N, int G, float* out, void* stream) {
    if (!proj || !xbc || !A_log || !Dp || !dt_bias || !state || !st || !out || H < 1 || V < 1 || N < 1 || G < 1 || H % G)
        return fail(B200SEQ_ERR_INVALID_ARG, "ssm_scan: bad arguments");
    if (N > 256) return fail(B200SEQ_ERR_UNSUPPORTED, "ssm_scan: state size %d > 256", N);
    if (st->B == 0 || st->T == 0) return 0;
    dim3 grid((V + 31) / 32, H, st->B);
    const size_t smem = ((size_t)2 * SSM_TT * N + 2 * SSM_TT) * sizeof(float);
    cudaStream_t cs = (cudaStream_t)stream;
#define SSM_LAUNCH(NPT) ssm_scan_kernel<NPT><<<grid, 32, smem, cs>>>(proj, ldp, z0, dt0, xbc, ldx, A_log, Dp, dt_bias, state, *st, H, V, N, G, out)
    if (N <= 16) SSM_LAUNCH(16);
    else if (N <= 32) SSM_LAUNCH(32);
    else if (N <= 64) SSM_LAUNCH(64);
    else if (N <= 128) SSM_LAUNCH(128);
    else SSM_LAUNCH(256);
#undef SSM_LAUNCH
    SEQ_LAUNCH_CHECK("ssm_scan");
    return 0;
}
