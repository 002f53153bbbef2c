// Recurrent mixers with a matrix state per head: S [key_dim, value_dim] in float, carried from
// token to token for each sequence.
//
//   gated delta rule (one decay per key channel):  S <- diag(g) S;  u = beta (v - S^T k);
//                                                  S <- S + k u^T;  o = S^T q
//   matrix memory with exponential gates:          m' = max(f + m, i);
//                                                  S <- e^(f + m - m') S + e^(i - m') k v^T  (n likewise with k alone);
//                                                  o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)
//
// Both are independent per column of S: a thread owns one column (key_dim floats in
// registers) of one (sequence, head) and walks the sequence's new tokens in order, so a
// prompt's rows and the same rows fed one by one are summed in the same order. The matrix
// memory keeps n as one more column (whose v is 1) and m as one more row, per column, so
// that no thread reads what another writes. q, k, gates of a few tokens at a time are staged
// in shared memory by the whole block.
//
// Before them: the short causal convolution with SiLU and the unit norm of q and k for the
// delta rule. After them: the per-head RMS norm with weight and sigmoid gate.
#include "common.cuh"

#define REC_TOKENS 8          // tokens staged per round

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoid_f(float x) { return x < 0.f ? x - log1pf(expf(x)) : -log1pf(expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------
// Short convolution + SiLU (+ unit norm). `proj` [rows, ld] holds, from column 0, the q
// channels (qk_heads x key_dim), the k channels (the same) and the v channels (heads x
// value_dim) before the convolution; `conv_w` [channels, taps] float, the last tap the current
// token's; `state` [slots, taps - 1, channels] the inputs of the tokens before the step.
// A warp owns one (row, head of q | k | v). q and k become x / sqrt(sum x^2 + 1e-6), q times
// q_scale. out [rows, channels] float.
__global__ void conv_unit_kernel(const float* __restrict__ proj, long ld, const float* __restrict__ conv_w,
                                 const float* __restrict__ state, const int* __restrict__ row_seq,
                                 const int* __restrict__ row_pos, const int* __restrict__ seq_row0,
                                 const int* __restrict__ seq_slot, float* __restrict__ out, int rows, int qk_heads,
                                 int heads, int key_dim, int value_dim, int taps, float q_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int units = 2 * qk_heads + heads;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * units) return;
    const int r = warp / units, u = warp % units;
    const int channels = 2 * qk_heads * key_dim + heads * value_dim;
    int c0, n;
    if (u < 2 * qk_heads) { c0 = u * key_dim; n = key_dim; }
    else { c0 = 2 * qk_heads * key_dim + (u - 2 * qk_heads) * value_dim; n = value_dim; }
    const int s = row_seq[r], pos = row_pos[r], inside = r - seq_row0[s];
    const float* st = state + (size_t)seq_slot[s] * (taps - 1) * channels;
    float ss = 0.f;
    for (int c = c0 + lane; c < c0 + n; c += 32) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;                 // tokens before this one
            if (back > pos) continue;                      // before the sequence's start
            float x;
            if (back <= inside) x = proj[(size_t)(r - back) * ld + c];
            else x = st[(size_t)(taps - 1 + inside - back) * channels + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        acc = silu_f(acc);
        out[(size_t)r * channels + c] = acc;
        ss = fmaf(acc, acc, ss);
    }
    if (u < 2 * qk_heads) {
        ss = warp_sum(ss);
        const float scale = (u < qk_heads ? q_scale : 1.0f) / sqrtf(ss + 1e-6f);
        __syncwarp();
        for (int c = c0 + lane; c < c0 + n; c += 32) out[(size_t)r * channels + c] *= scale;
    }
}

extern "C" int cml_conv_unit(const float* proj, long ld, const float* conv_w, const float* state, const int* row_seq,
                             const int* row_pos, const int* seq_row0, const int* seq_slot, float* out, int rows, int qk_heads,
                             int heads, int key_dim, int value_dim, int taps, float q_scale, void* stream) {
    if (rows <= 0) return 0;
    if (taps < 1) return CML_ERR_BAD_SIZE;
    const long warps = (long)rows * (2 * qk_heads + heads);
    launch_pdl(conv_unit_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, proj, ld, conv_w, state,
               row_seq, row_pos, seq_row0, seq_slot, out, rows, qk_heads, heads, key_dim, value_dim, taps, q_scale);
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// Gated delta rule. qkv [rows, ldq]: unit q (qk_heads x D), unit k, v (heads x Dv) from
// conv_unit_kernel. beta_in [rows, ldb] at column beta_col + head: before the sigmoid.
// decay_in [rows, ldd] (heads x D): before dt_bias; g = exp(-exp(a_log[head]) softplus(x + dt_bias)).
// state [slots, heads, D, Dv]. out [rows, heads x Dv] float, S^T q.
template <int DMAX>
__global__ void __launch_bounds__(128) delta_scan_kernel(
        const float* __restrict__ qkv, long ldq, const float* __restrict__ beta_in, long ldb, int beta_col,
        const float* __restrict__ decay_in, long ldd, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
        float* __restrict__ state, const int* __restrict__ seq_row0, const int* __restrict__ seq_new,
        const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ out, int heads,
        int qk_heads, int D, int Dv) {
    __shared__ float sq[REC_TOKENS][DMAX], sk[REC_TOKENS][DMAX], sg[REC_TOKENS][DMAX];
    __shared__ float sv[REC_TOKENS][128], sbeta[REC_TOKENS];
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, hd = blockIdx.y, g = hd / (heads / qk_heads);
    const int c = blockIdx.z * blockDim.x + threadIdx.x;
    const bool live = c < Dv;
    const int row0 = seq_row0[s], n = seq_new[s];
    float* st = state + (((size_t)seq_slot[s] * heads + hd) * D) * Dv + (live ? c : 0);
    float S[DMAX];
    const bool fresh = seq_start[s] == 0;
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (d < D && live && !fresh) ? st[(size_t)d * Dv] : 0.f;
    const float a_rate = expf(a_log[hd]);
    const int vcol = 2 * qk_heads * D + hd * Dv;
    for (int t0 = 0; t0 < n; t0 += REC_TOKENS) {
        const int nt = min(REC_TOKENS, n - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * D; i += blockDim.x) {
            const int t = i / D, d = i % D;
            const size_t r = (size_t)(row0 + t0 + t);
            sq[t][d] = qkv[r * ldq + g * D + d];
            sk[t][d] = qkv[r * ldq + (qk_heads + g) * D + d];
            sg[t][d] = expf(-a_rate * softplus_f(decay_in[r * ldd + hd * D + d] + dt_bias[hd * D + d]));
        }
        for (int i = threadIdx.x; i < nt * (int)blockDim.x; i += blockDim.x) {
            const int t = i / blockDim.x, cc = blockIdx.z * blockDim.x + i % blockDim.x;
            sv[t][i % blockDim.x] = cc < Dv ? qkv[(size_t)(row0 + t0 + t) * ldq + vcol + cc] : 0.f;
        }
        if (threadIdx.x < nt) sbeta[threadIdx.x] = sigmoid_f(beta_in[(size_t)(row0 + t0 + threadIdx.x) * ldb + beta_col + hd]);
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            float dot = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; ++d)
                if (d < D) { S[d] *= sg[t][d]; dot = fmaf(S[d], sk[t][d], dot); }
            const float u = sbeta[t] * (sv[t][threadIdx.x] - dot);
            float o = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; ++d)
                if (d < D) { S[d] = fmaf(sk[t][d], u, S[d]); o = fmaf(S[d], sq[t][d], o); }
            if (live) out[(size_t)(row0 + t0 + t) * heads * Dv + hd * Dv + c] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
            if (d < D) st[(size_t)d * Dv] = S[d];
    }
}

extern "C" int cml_delta_scan(const float* qkv, long ldq, const float* beta_in, long ldb, int beta_col, const float* decay_in,
                              long ldd, const float* a_log, const float* dt_bias, float* state, const int* seq_row0,
                              const int* seq_new, const int* seq_start, const int* seq_slot, float* out, int n_seqs, int heads,
                              int qk_heads, int D, int Dv, void* stream) {
    if (n_seqs <= 0) return 0;
    if (D < 1 || D > 256 || Dv < 1 || heads % qk_heads) return CML_ERR_BAD_SIZE;
    const int threads = Dv <= 32 ? 32 : (Dv <= 64 ? 64 : 128);
    dim3 grid(n_seqs, heads, (Dv + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
#define DS_CASE(DM)                                                                                                        \
    if (D <= DM) {                                                                                                         \
        launch_pdl(delta_scan_kernel<DM>, grid, dim3(threads), 0, s, qkv, ldq, beta_in, ldb, beta_col, decay_in, ldd, a_log,  \
                   dt_bias, state, seq_row0, seq_new, seq_start, seq_slot, out, heads, qk_heads, D, Dv);                   \
        return cml_launch_status();                                                                                        \
    }
    DS_CASE(16) DS_CASE(32) DS_CASE(64) DS_CASE(128) DS_CASE(256)
#undef DS_CASE
    return CML_ERR_BAD_SIZE;
}

// ------------------------------------------------------------------------------------
// Matrix memory. proj [rows, ld] float holds q at q_col (heads x D), k at k_col, v at v_col
// (heads x Dv), and the gate inputs at i_col + head and f_col + head (before bias and cap).
// state [slots, heads, D + 1, Dv + 1]: S with n as column Dv, and m as row D (one copy per
// column). out [rows, heads, Dv + 2] float: S^T q per column, then n . q, then m after the token.
template <int DMAX>
__global__ void __launch_bounds__(128) memory_scan_kernel(
        const float* __restrict__ proj, long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
        const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
        float* __restrict__ state, const int* __restrict__ seq_row0, const int* __restrict__ seq_new,
        const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ out, int heads, int D,
        int Dv) {
    __shared__ float sq[REC_TOKENS][DMAX], sk[REC_TOKENS][DMAX];
    __shared__ float sv[REC_TOKENS][128], si[REC_TOKENS], sf[REC_TOKENS];
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, hd = blockIdx.y;
    const int c = blockIdx.z * blockDim.x + threadIdx.x;
    const int cols = Dv + 1;
    const bool live = c < cols;
    const int row0 = seq_row0[s], n = seq_new[s];
    float* st = state + (((size_t)seq_slot[s] * heads + hd) * (D + 1)) * cols + (live ? c : 0);
    const bool fresh = seq_start[s] == 0;
    float S[DMAX];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (d < D && live && !fresh) ? st[(size_t)d * cols] : 0.f;
    float m = (live && !fresh) ? st[(size_t)D * cols] : 0.f;
    for (int t0 = 0; t0 < n; t0 += REC_TOKENS) {
        const int nt = min(REC_TOKENS, n - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * D; i += blockDim.x) {
            const int t = i / D, d = i % D;
            const size_t r = (size_t)(row0 + t0 + t);
            sq[t][d] = proj[r * ld + q_col + hd * D + d] * q_scale;
            sk[t][d] = proj[r * ld + k_col + hd * D + d];
        }
        for (int i = threadIdx.x; i < nt * (int)blockDim.x; i += blockDim.x) {
            const int t = i / blockDim.x, cc = blockIdx.z * blockDim.x + i % blockDim.x;
            sv[t][i % blockDim.x] = cc < Dv ? proj[(size_t)(row0 + t0 + t) * ld + v_col + hd * Dv + cc] : 1.0f;
        }
        if (threadIdx.x < nt) {
            const size_t r = (size_t)(row0 + t0 + threadIdx.x);
            si[threadIdx.x] = cap * tanhf((proj[r * ld + i_col + hd] + i_bias[hd]) / cap);
            sf[threadIdx.x] = logsigmoid_f(cap * tanhf((proj[r * ld + f_col + hd] + f_bias[hd]) / cap));
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float fm = sf[t] + m;
            const float m_new = fmaxf(fm, si[t]);
            const float a = expf(fm - m_new);
            const float bv = expf(si[t] - m_new) * sv[t][threadIdx.x];
            m = m_new;
            float o = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; ++d)
                if (d < D) { S[d] = fmaf(a, S[d], bv * sk[t][d]); o = fmaf(S[d], sq[t][d], o); }
            if (live) {
                float* orow = out + ((size_t)(row0 + t0 + t) * heads + hd) * (Dv + 2);
                orow[c] = o;
                if (c == Dv) orow[Dv + 1] = m;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
            if (d < D) st[(size_t)d * cols] = S[d];
        st[(size_t)D * cols] = m;
    }
}

extern "C" int cml_memory_scan(const float* proj, long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                               const float* i_bias, const float* f_bias, float cap, float q_scale, float* state,
                               const int* seq_row0, const int* seq_new, const int* seq_start, const int* seq_slot, float* out,
                               int n_seqs, int heads, int D, int Dv, void* stream) {
    if (n_seqs <= 0) return 0;
    if (D < 1 || D > 256 || Dv < 1) return CML_ERR_BAD_SIZE;
    const int cols = Dv + 1;
    const int threads = cols <= 32 ? 32 : (cols <= 64 ? 64 : 128);
    dim3 grid(n_seqs, heads, (cols + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
#define MS_CASE(DM)                                                                                                        \
    if (D <= DM) {                                                                                                         \
        launch_pdl(memory_scan_kernel<DM>, grid, dim3(threads), 0, s, proj, ld, q_col, k_col, v_col, i_col, f_col, i_bias,    \
                   f_bias, cap, q_scale, state, seq_row0, seq_new, seq_start, seq_slot, out, heads, D, Dv);                \
        return cml_launch_status();                                                                                        \
    }
    MS_CASE(16) MS_CASE(32) MS_CASE(64) MS_CASE(128) MS_CASE(256)
#undef MS_CASE
    return CML_ERR_BAD_SIZE;
}

// ------------------------------------------------------------------------------------
// After a scan: per (row, head) o = raw / den (den = max(|n . q|, exp(-m)) + 1e-6 where the
// raw rows carry them, else 1), y = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate), written in
// the compute type for the output projection. A warp owns one (row, head). raw [rows, heads, ldh]
// with ldh = Dv (+ 2 with a denominator); w [Dv] shared by the heads (w_head_stride 0) or
// [heads x Dv]; gate [rows, ldg] at column gate_col + head * Dv.
template <typename TO>
__global__ void head_norm_gate_kernel(const float* __restrict__ raw, int ldh, int with_den, const float* __restrict__ w,
                                      int w_head_stride, const float* __restrict__ gate, long ldg, int gate_col,
                                      TO* __restrict__ out, int rows, int heads, int Dv, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * heads) return;
    const int r = warp / heads, hd = warp % heads;
    const float* x = raw + ((size_t)r * heads + hd) * ldh;
    float inv = 1.0f;
    if (with_den) inv = 1.0f / (fmaxf(fabsf(x[Dv]), expf(-x[Dv + 1])) + 1e-6f);
    float ss = 0.f;
    for (int c = lane; c < Dv; c += 32) {
        const float o = x[c] * inv;
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float scale = inv / sqrtf(ss / (float)Dv + eps);
    const float* wv = w + (size_t)hd * w_head_stride;
    const float* gt = gate + (size_t)r * ldg + gate_col + hd * Dv;
    TO* o = out + ((size_t)r * heads + hd) * Dv;
    for (int c = lane; c < Dv; c += 32) o[c] = from_f32<TO>(x[c] * scale * wv[c] * sigmoid_f(gt[c]));
}

extern "C" int cml_head_norm_gate(const float* raw, int ldh, int with_den, const float* w, int w_head_stride, const float* gate,
                                  long ldg, int gate_col, void* out, int out_dtype, int rows, int heads, int Dv, float eps,
                                  void* stream) {
    if (rows <= 0) return 0;
    const long warps = (long)rows * heads;
    dim3 grid((unsigned)((warps + 3) / 4));
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == CML_DTYPE_F32)
        launch_pdl(head_norm_gate_kernel<float>, grid, dim3(128), 0, s, raw, ldh, with_den, w, w_head_stride, gate, ldg, gate_col,
                   (float*)out, rows, heads, Dv, eps);
    else if (out_dtype == CML_DTYPE_BF16)
        launch_pdl(head_norm_gate_kernel<bf16>, grid, dim3(128), 0, s, raw, ldh, with_den, w, w_head_stride, gate, ldg, gate_col,
                   (bf16*)out, rows, heads, Dv, eps);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
