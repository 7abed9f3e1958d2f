// seq_ssm.cu -- selective state-space recurrence (scalar decay per head, state N x V per head) over a flat mixed batch.
//
// One block per (tile of value columns, head, segment of tokens).  A value column's state (N floats) is spread over NL lanes
// (NL = 1, 2, 4 or 8, at most 32 floats per lane, so it stays in registers); a warp covers 32 / NL columns.  The tokens of a
// segment are walked in order; x, z, B, C, the step sizes and the decays of a tile of SSM_TT tokens are staged in shared memory
// with coalesced loads, the outputs of the tile leave through shared memory too.  Step sizes, decays and the state are f32.
//
// Short steps (T <= SSM_SEG: decode, small portions): one launch, a segment is an entry's whole portion, the state comes from and
// returns to the sequence's slot (read as zero for a new sequence).
// Long steps: every entry is cut into segments of SSM_SEG tokens that run in parallel, in three launches:
//   A  each segment runs the recurrence from a zero state -> its local end state E and the sum of its log-decays
//   B  per entry, in order: start[s] = S;  S = exp(sum log-decay of s) * S + E[s]   (elementwise; the last S goes to the slot)
//   C  each segment runs again from start[s] and writes the outputs
// which costs twice the arithmetic of the plain recurrence and removes the dependence on the portion's length.
#include "seq_common.cuh"

namespace b200seq {

constexpr int SSM_TT = 16;     // tokens per staged tile
constexpr int SSM_SEG = 128;   // tokens per parallel segment
constexpr int SSM_WARPS = 8;
enum { SSM_DIRECT = 0, SSM_LOCAL = 1, SSM_FINAL = 2 };

struct SsmArgs {
    const float* proj;
    int64_t ldp;
    int z0, dt0;
    const float* xbc;
    int64_t ldx;
    const float *A_log, *Dp, *dt_bias;
    float* state;     // [slots][H][N][V]
    float* seg_state; // [segments][H][N][V]   (E after pass A, start state after pass B)
    float* seg_logdec;  // [segments][H]
    float* out;
    int H, V, N, G, NL, seg_len;
};

// segment `idx` of the step: entry, first token row, token count, whether it is the entry's first
__device__ __forceinline__ bool ssm_find_segment(const b200seq_step& st, int idx, int seg_len, int& e, int& row0, int& len) {
    int acc = 0;
    for (e = 0; e < st.B; ++e) {
        const int s0 = st.ent_start[e], n = st.ent_start[e + 1] - s0;
        const int ns = (n + seg_len - 1) / seg_len;
        if (idx < acc + ns) {
            const int local = idx - acc;
            row0 = s0 + local * seg_len;
            len = min(seg_len, n - local * seg_len);
            return true;
        }
        acc += ns;
    }
    return false;
}

// NPL: state floats per lane.  Lane -> (sub = lane / cpw, col = lane % cpw), cpw = 32 / NL; the lane holds n = sub * NPL + i.
template <int NPL, int MODE>
__global__ void __launch_bounds__(SSM_WARPS * 32) ssm_kernel(const SsmArgs a, const b200seq_step st) {
    extern __shared__ __align__(16) float sm[];
    const int H = a.H, V = a.V, N = a.N, NL = a.NL;
    const int cpw = 32 / NL, cols = SSM_WARPS * cpw;       // value columns of this block (NL, cpw, cols and NPL are powers of two)
    const int cols_shift = 31 - __clz(cols), npl_shift = 31 - __clz(NPL), nn_shift = npl_shift + (31 - __clz(NL));
    const int nstride = NPL + 4;                           // padded chunk of one sub-lane (conflict-free 16-byte reads)
    const int nrow = NL * nstride;
    float* Bs = sm;                          // [SSM_TT][nrow]
    float* Cs = Bs + SSM_TT * nrow;          // [SSM_TT][nrow]
    float* xs = Cs + SSM_TT * nrow;          // [SSM_TT][cols]   (outputs replace x)
    float* zs = xs + SSM_TT * cols;          // [SSM_TT][cols]
    float* dts = zs + SSM_TT * cols;         // [SSM_TT]
    float* dec = dts + SSM_TT;               // [SSM_TT]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane / cpw, cl = warp * cpw + lane % cpw;
    const int v0 = blockIdx.x * cols, v = v0 + cl;
    const int h = blockIdx.y;
    int e, row0, len;
    if (MODE == SSM_DIRECT) {
        e = blockIdx.z;
        row0 = st.ent_start[e];
        len = st.ent_start[e + 1] - row0;
    } else if (!ssm_find_segment(st, blockIdx.z, a.seg_len, e, row0, len)) {
        return;
    }
    const bool live = v < V;
    const int g = h / (H / a.G);
    const int inner = H * V;
    float S[NPL];
    const float* init = nullptr;
    if (MODE == SSM_DIRECT) init = st.ent_pos0[e] == 0 ? nullptr : a.state + ((int64_t)st.ent_slot[e] * H + h) * N * V;
    if (MODE == SSM_FINAL) init = a.seg_state + ((int64_t)blockIdx.z * H + h) * N * V;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int n = sub * NPL + i;
        S[i] = (init && live && n < N) ? init[(int64_t)n * V + v] : 0.f;
    }
    const float negA = -expf(a.A_log[h]);
    const float dtb = a.dt_bias[h], Dh = a.Dp[h];
    float logdec = 0.f;   // thread 0 only (pass A)
    for (int i0 = 0; i0 < len; i0 += SSM_TT) {
        const int nt = min(SSM_TT, len - i0);
        __syncthreads();
        for (int idx = tid; idx < (nt << nn_shift); idx += blockDim.x) {
            const int tt = idx >> nn_shift, n = idx & ((1 << nn_shift) - 1);
            const int at = tt * nrow + (n >> npl_shift) * nstride + (n & (NPL - 1));
            float b = 0.f, c = 0.f;
            if (n < N) {
                const float* r = a.xbc + (int64_t)(row0 + i0 + tt) * a.ldx + inner + (int64_t)g * N + n;
                b = r[0];
                if (MODE != SSM_LOCAL) c = r[(int64_t)a.G * N];
            }
            Bs[at] = b;
            Cs[at] = c;
        }
        for (int idx = tid; idx < (nt << cols_shift); idx += blockDim.x) {
            const int tt = idx >> cols_shift, c = idx & (cols - 1);
            const int64_t row = row0 + i0 + tt;
            const bool in = v0 + c < V;
            xs[idx] = in ? a.xbc[row * a.ldx + (int64_t)h * V + v0 + c] : 0.f;
            if (MODE != SSM_LOCAL) zs[idx] = in ? a.proj[row * a.ldp + a.z0 + (int64_t)h * V + v0 + c] : 0.f;
        }
        if (tid < nt) {
            const float dt = softplusf_acc(a.proj[(int64_t)(row0 + i0 + tid) * a.ldp + a.dt0 + h] + dtb);
            dts[tid] = dt;
            dec[tid] = expf(negA * dt);
        }
        __syncthreads();
        if (MODE == SSM_LOCAL && tid == 0)
            for (int tt = 0; tt < nt; ++tt) logdec += negA * dts[tt];
        for (int tt = 0; tt < nt; ++tt) {
            const float x = xs[tt * cols + cl];
            const float dA = dec[tt], dtx = dts[tt] * x;
            const float4* Bt = reinterpret_cast<const float4*>(Bs + tt * nrow + sub * nstride);
            const float4* Ct = reinterpret_cast<const float4*>(Cs + tt * nrow + sub * nstride);
            float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
            for (int i = 0; i < NPL / 4; ++i) {
                const float4 b = Bt[i];
                S[4 * i] = fmaf(dA, S[4 * i], dtx * b.x);
                S[4 * i + 1] = fmaf(dA, S[4 * i + 1], dtx * b.y);
                S[4 * i + 2] = fmaf(dA, S[4 * i + 2], dtx * b.z);
                S[4 * i + 3] = fmaf(dA, S[4 * i + 3], dtx * b.w);
                if (MODE != SSM_LOCAL) {
                    const float4 c = Ct[i];
                    y0 = fmaf(S[4 * i], c.x, y0), y1 = fmaf(S[4 * i + 1], c.y, y1), y2 = fmaf(S[4 * i + 2], c.z, y2), y3 = fmaf(S[4 * i + 3], c.w, y3);
                }
            }
            if (MODE != SSM_LOCAL) {
                float y = (y0 + y1) + (y2 + y3);
                for (int o = cpw; o < 32; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                __syncwarp();
                if (sub == 0) xs[tt * cols + cl] = fmaf(Dh, x, y) * siluf_acc(zs[tt * cols + cl]);   // x of this token is consumed
            }
        }
        if (MODE != SSM_LOCAL) {
            __syncthreads();
            for (int idx = tid; idx < (nt << cols_shift); idx += blockDim.x) {
                const int tt = idx >> cols_shift, c = idx & (cols - 1);
                if (v0 + c < V) a.out[(int64_t)(row0 + i0 + tt) * inner + (int64_t)h * V + v0 + c] = xs[idx];
            }
        }
    }
    if (MODE == SSM_FINAL) return;
    float* dst = MODE == SSM_DIRECT ? a.state + ((int64_t)st.ent_slot[e] * H + h) * N * V : a.seg_state + ((int64_t)blockIdx.z * H + h) * N * V;
    if (live) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int n = sub * NPL + i;
            if (n < N) dst[(int64_t)n * V + v] = S[i];
        }
    }
    if (MODE == SSM_LOCAL && tid == 0 && blockIdx.x == 0) a.seg_logdec[(int64_t)blockIdx.z * H + h] = logdec;
}

// pass B: one thread per (entry, head, n, v); walks the entry's segments in order
__global__ void ssm_combine_kernel(const SsmArgs a, const b200seq_step st) {
    const int64_t per = (int64_t)a.H * a.N * a.V;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int e = blockIdx.y;
    if (idx >= per) return;
    const int h = (int)(idx / ((int64_t)a.N * a.V));
    int seg0 = 0;
    for (int i = 0; i < e; ++i) seg0 += (st.ent_start[i + 1] - st.ent_start[i] + a.seg_len - 1) / a.seg_len;
    const int ns = (st.ent_start[e + 1] - st.ent_start[e] + a.seg_len - 1) / a.seg_len;
    float* slot = a.state + (int64_t)st.ent_slot[e] * per + idx;
    float S = st.ent_pos0[e] == 0 ? 0.f : *slot;
    for (int s = 0; s < ns; ++s) {
        float* p = a.seg_state + (int64_t)(seg0 + s) * per + idx;
        const float E = *p;
        *p = S;
        S = fmaf(expf(a.seg_logdec[(int64_t)(seg0 + s) * a.H + h]), S, E);
    }
    *slot = S;
}

template <int NPL, int MODE>
static cudaError_t ssm_launch(const SsmArgs& a, const b200seq_step& st, int nz, cudaStream_t cs) {
    const int cpw = 32 / a.NL, cols = SSM_WARPS * cpw;
    const size_t smem = ((size_t)2 * SSM_TT * a.NL * (NPL + 4) + 2 * SSM_TT * cols + 2 * SSM_TT + 4) * sizeof(float);
    dim3 grid((a.V + cols - 1) / cols, a.H, nz);
    ssm_kernel<NPL, MODE><<<grid, SSM_WARPS * 32, smem, cs>>>(a, st);
    return cudaGetLastError();
}

}  // namespace b200seq

using namespace b200seq;

extern "C" size_t b200seq_ssm_scratch_floats(int T, int B, int H, int V, int N) {
    if (T <= SSM_SEG) return 0;
    const size_t segs = (size_t)(T + SSM_SEG - 1) / SSM_SEG + (size_t)B;
    return segs * ((size_t)H * N * V + H);
}

extern "C" int b200seq_ssm_scan(const float* proj, int64_t ldp, int z0, int dt0, const float* xbc, int64_t ldx, const float* A_log, const float* Dp,
                                const float* dt_bias, float* state, const b200seq_step* st, int H, int V, int N, int G, float* out, float* scratch,
                                size_t scratch_floats, void* stream) {
    if (!proj || !xbc || !A_log || !Dp || !dt_bias || !state || !st || !out || H < 1 || V < 1 || N < 1 || G < 1 || H % G)
        return fail(B200SEQ_ERR_INVALID_ARG, "ssm_scan: bad arguments");
    if (N > 256) return fail(B200SEQ_ERR_UNSUPPORTED, "ssm_scan: state size %d > 256", N);
    if (st->B == 0 || st->T == 0) return 0;
    cudaStream_t cs = (cudaStream_t)stream;
    SsmArgs a{proj, ldp, z0, dt0, xbc, ldx, A_log, Dp, dt_bias, state, nullptr, nullptr, out, H, V, N, G, 1, SSM_SEG};
    const bool small = N <= 16;
    const int npl = small ? 16 : 32;
    while (a.NL * npl < N) a.NL *= 2;
    const size_t need = b200seq_ssm_scratch_floats(st->T, st->B, H, V, N);
    cudaError_t e;
    if (need == 0 || !scratch || scratch_floats < need) {   // one launch: every entry's portion in order
        e = small ? ssm_launch<16, SSM_DIRECT>(a, *st, st->B, cs) : ssm_launch<32, SSM_DIRECT>(a, *st, st->B, cs);
        if (e != cudaSuccess) return cuda_status(e, "ssm_scan");
        count_launch();
        return 0;
    }
    const int segs = (st->T + SSM_SEG - 1) / SSM_SEG + st->B;   // upper bound of the step's segment count
    a.seg_state = scratch;
    a.seg_logdec = scratch + (size_t)segs * H * N * V;
    e = small ? ssm_launch<16, SSM_LOCAL>(a, *st, segs, cs) : ssm_launch<32, SSM_LOCAL>(a, *st, segs, cs);
    if (e != cudaSuccess) return cuda_status(e, "ssm_scan local pass");
    const int64_t per = (int64_t)H * N * V;
    ssm_combine_kernel<<<dim3((unsigned)((per + 255) / 256), st->B), 256, 0, cs>>>(a, *st);
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_status(e, "ssm_scan combine pass");
    e = small ? ssm_launch<16, SSM_FINAL>(a, *st, segs, cs) : ssm_launch<32, SSM_FINAL>(a, *st, segs, cs);
    if (e != cudaSuccess) return cuda_status(e, "ssm_scan final pass");
    count_launch(3);
    return 0;
}
