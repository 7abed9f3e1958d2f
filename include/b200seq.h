/*
 * b200seq.h -- C ABI of libb200seq.so: dense (bfloat16-weight) linear layers and the sequence operators of
 * layer-list models on B200 (sm_100a): multi-stream residual mixing with grouped RMS norm, short causal
 * convolutions with carried state, chunk/window-masked attention over a paged KV pool, the selective
 * state-space recurrence with per-slot state, gated feed-forward activations, arg-max sampling.
 *
 * It sits beside libb200q (include/b200q.h), which holds the quantized linear layer; the conventions are
 * the same:
 *   - every function returns 0 or a negative status; b200seq_last_error() gives the message;
 *   - `stream` is a cudaStream_t passed as void*;
 *   - no allocation, no host synchronisation, no host scalar that changes from step to step: a step of
 *     fixed token count is CUDA-graph capturable;
 *   - no CPU fallback.
 *
 * A step is a flat batch of T tokens belonging to B entries (one entry = the next tokens of one request,
 * a prompt portion or a single decoded token).  The int32 device arrays every sequence operator reads:
 *   tok_ent[T]        entry of each token
 *   tok_pos[T]        position of each token in its sequence (from 0)
 *   ent_start[B + 1]  first token row of each entry (prefix sums of the portion lengths)
 *   ent_slot[B]       state slot of the entry's request
 *   ent_pos0[B]       position of the entry's first token (0 = a new sequence: carried state reads as zero)
 *   block_table[B][max_blocks]  KV pages of the entry's request
 * Activations that feed a linear layer are written in `act` dtype (B200SEQ_F32 or B200SEQ_BF16); everything
 * else (residual streams, norms, scores, recurrent state, KV pool) is float32.
 */
#ifndef B200SEQ_H
#define B200SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200SEQ_OK 0
#define B200SEQ_ERR_INVALID_ARG (-1)
#define B200SEQ_ERR_UNSUPPORTED (-2)
#define B200SEQ_ERR_CUDA (-3)

#define B200SEQ_F32 0
#define B200SEQ_BF16 2

/* b200seq_causal_conv modes */
#define B200SEQ_CONV_RESIDUAL 1 /* out = x + conv(x) */
#define B200SEQ_CONV_SILU 2     /* out = silu(conv(x) + bias) */

/* b200seq_linear paths */
#define B200SEQ_PATH_AUTO 0
#define B200SEQ_PATH_ROWS 1   /* weight-streaming warp-per-row kernel (few tokens) */
#define B200SEQ_PATH_TILED 2  /* float32 FMA tiles (any M, exact 32-bit arithmetic) */
#define B200SEQ_PATH_TC 3     /* tcgen05 tensor-core tiles (bf16 activations) */

typedef struct b200seq_step {
    const int32_t* tok_ent;
    const int32_t* tok_pos;
    const int32_t* ent_start;
    const int32_t* ent_slot;
    const int32_t* ent_pos0;
    const int32_t* block_table;
    int32_t T, B, max_blocks, block_size;
} b200seq_step;

const char* b200seq_last_error(void);
int b200seq_version(void);
int64_t b200seq_launch_count(void);
/* bit 0: a KV position fell outside its block table; bit 1: a bounded wait of the tensor-core GEMM ran out */
int b200seq_error_flags(int* flags_out);

/* X[t][s][:] = table[ids[t]][:] * scale for every stream s.  table: bf16 [V, W]; X: f32 [T, S, W]. */
int b200seq_embed_streams(const void* table_bf16, const int32_t* ids, float scale, int T, int S, int W, float* X, void* stream);

/* Stream update and collapse around a sublayer, one block per row r (token t = rows ? rows[r] : r):
 *   if y:      X[t][j] <- sum_s post[S + s * S + j] * X[t][s] + post[j] * y[t]      (post = out[S] | mix[S][S], mix indexed [from][to])
 *   if norm_w: u = sum_s in_w[s] * X[t][s];  out[r] = group_rms(u, groups, eps) * norm_w
 * y: f32 [T, W] or null; out: [R, W] in out_dtype. */
int b200seq_hc_norm(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                    const int32_t* rows, int R, void* out, int out_dtype, void* stream);

/* The same followed by the sublayer's carried convolution (mode B200SEQ_CONV_RESIDUAL, no bias) in one kernel, for steps in which every
 * entry brings exactly one token (st->T == st->B, all rows): out[t] = h + conv(h), conv_state[slot][taps-1][W] read and shifted. */
int b200seq_hc_norm_conv(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                         const float* conv_w, float* conv_state, const b200seq_step* st, int taps, void* out, int out_dtype, void* stream);

/* Per-channel causal convolution over time with the last taps-1 inputs of every sequence carried in
 * state[slot][taps-1][C] (f32; read as zero when ent_pos0 == 0, rewritten for every entry of the step).
 * x: f32 rows of stride ldx; w: f32 [C, taps] (last column = current token); bias f32 [C] or null. */
int b200seq_causal_conv(const float* x, int64_t ldx, const float* w, const float* bias, float* state, const b200seq_step* st, int C, int taps, int mode,
                        void* out, int out_dtype, int64_t ldo, void* stream);

/* out[t] = group_rms(x[t], groups, eps) * w   (x f32 [T, D] stride ldx; out act dtype [T, D]) */
int b200seq_group_rmsnorm(const float* x, int64_t ldx, const float* w, int T, int D, int groups, float eps, void* out, int out_dtype, void* stream);

/* gu: f32 [T, 2F] = gate | up (interleaved = 0) or gate 0, up 0, gate 1, up 1, ... (interleaved = 1).
 * g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + up_shift) */
int b200seq_gated_act(const float* gu, int64_t ldg, int T, int F, float limit, float alpha, float up_shift, int interleaved, void* out, int out_dtype,
                      void* stream);

/* y[M, N] (f32, stride ldy) = x[M, K] (f32 or bf16, stride ldx) . w[N, K]^T (bf16, contiguous) */
int b200seq_linear(const void* x, int x_dtype, int64_t ldx, const void* w_bf16, int M, int N, int K, float* y, int64_t ldy, int path, void* stream);

/* Fused gate|up projection + gated activation: w_il is the stacked weight [2F, K] with rows alternating (gate 0, up 0, gate 1, up 1, ...);
 * out[M, F] (act dtype, stride ldo) = gated_act(x . w_il^T) with the formula of b200seq_gated_act.  The [M, 2F] product is never written.
 * M <= 8: weight-streaming rows (f32 or bf16 activations); more rows: the tensor-core path, which needs bf16 activations, K % 8 == 0 and
 * 16-byte aligned rows (B200SEQ_ERR_UNSUPPORTED otherwise). */
int b200seq_linear_gated(const void* x, int x_dtype, int64_t ldx, const void* w_il_bf16, int M, int F, int K, float limit, float alpha, float up_shift,
                         void* out, int out_dtype, int64_t ldo, void* stream);

/* Attention over a paged f32 KV pool (kpool [blocks][block_size][G][D], vpool [..][G][V]).
 * qkvg: f32 [T, ld] = q (H*D) | k (G*D) | v (G*V) | gate (H, only if gated).
 * prep: q and k are divided per head by their RMS over D when qk_eps >= 0 (q in place), k and v go to the pool.
 * attend: token at position i sees j <= i with floor(j / chunk) == floor(i / chunk) (chunk > 0) and i - j < window (window > 0);
 *         softmax in f32, output times sigmoid(gate) when gated, written in act dtype to out [T, H*V]. */
int b200seq_attn_prep(float* qkvg, int64_t ld, const b200seq_step* st, float* kpool, float* vpool, int H, int G, int D, int V, float qk_eps, void* stream);
size_t b200seq_attn_scratch_floats(int T, int B, int H, int G, int V, int max_keys);
/* scratch: f32 work area of b200seq_attn_scratch_floats(...) floats (max_keys = the most keys a token can see) or null: with it, steps of
 * few tokens split the keys of a row among several blocks and merge the partial soft-max results. */
int b200seq_attn(const float* qkvg, int64_t ld, const b200seq_step* st, const float* kpool, const float* vpool, int H, int G, int D, int V, float scale,
                 int chunk, int window, int gated, void* out, int out_dtype, float* scratch, size_t scratch_floats, void* stream);

/* Selective state-space recurrence, per head h (group g = h / (H / G)), state[slot][H][N][V] f32 carried per sequence:
 *   dt = softplus(dt_raw + dt_bias[h]);  S <- exp(-exp(A_log[h]) * dt) * S + dt * B x^T;  y = S^T C + D[h] * x;  out = y * silu(z)
 * proj: f32 rows (stride ldp) with z at column z0 (H*V) and dt_raw at column dt0 (H);
 * xbc:  f32 rows (stride ldx) = x (H*V) | B (G*N) | C (G*N), already convolved and activated.  out: f32 [T, H*V].
 * scratch: f32 work area of b200seq_ssm_scratch_floats(T, B, ...) floats or null.  With it, steps of many tokens cut every portion into
 * segments that run in parallel (local pass, in-order combine, final pass); without it (or for short steps) each portion is one
 * sequential walk.  Both give the same result up to rounding. */
size_t b200seq_ssm_scratch_floats(int T, int B, int H, int V, int N);
int b200seq_ssm_scan(const float* proj, int64_t ldp, int z0, int dt0, const float* xbc, int64_t ldx, const float* A_log, const float* Dp, const float* dt_bias,
                     float* state, const b200seq_step* st, int H, int V, int N, int G, float* out, float* scratch, size_t scratch_floats, void* stream);

/* ids[r] = argmax_v logits[r][v] (first maximum) */
int b200seq_argmax(const float* logits, int R, int V, int32_t* ids, void* stream);

#ifdef __cplusplus
}
#endif
#endif
