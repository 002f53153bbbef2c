// Softmax attention over a sliding window of the paged cache, without rotation, for mixers
// whose keys and values may differ in size: per-head RMS norm of q and k, a penalty on the
// distance between query and key, an output gate.
//
//   score(i, j) = (q_i . k_j) scale - r1[head] ln(1 + r2[head] (i - j)),   0 <= i - j < window
//
// Two kernels. The first normalises q and k (weight per channel, shared by the heads), keeps
// q in the compute type and writes k and v into their pages. The second gives one warp to
// every (row, head): lanes take keys for the scores (all in float), then columns of the
// values; the softmax runs online over rounds of 32 keys, from the oldest visible key to the
// row's own, whether the row came with a prompt or alone.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_w(float x) { return 1.0f / (1.0f + expf(-x)); }

// proj [rows, ld] float: q (heads x D) at column 0, k (kv_heads x D), v (kv_heads x Dv).
// q_out [rows, heads x D]; pages [pages, kv_heads, 64, D | Dv]; table [seqs, max_blocks].
template <typename T, typename TW>
__global__ void qk_norm_kv_write_kernel(const float* __restrict__ proj, long ld, const TW* __restrict__ q_w,
                                        const TW* __restrict__ k_w, int qk_norm, float eps, const int* __restrict__ row_seq,
                                        const int* __restrict__ row_pos, const int* __restrict__ table, int max_blocks,
                                        T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int rows,
                                        int heads, int kv_heads, int D, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    const int units = heads + 2 * kv_heads;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * units) return;
    const int r = warp / units, u = warp % units;
    const float* x = proj + (size_t)r * ld;
    if (u < heads) {                                            // a query head
        x += u * D;
        float scale = 1.0f;
        if (qk_norm) {
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(x[c], x[c], ss);
            scale = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        T* o = q_out + ((size_t)r * heads + u) * D;
        for (int c = lane; c < D; c += 32) o[c] = from_f32<T>(qk_norm ? x[c] * scale * to_f32(q_w[c]) : x[c]);
        return;
    }
    const int pos = row_pos[r];
    const int page = table[(size_t)row_seq[r] * max_blocks + pos / CML_PAGE];
    if (page < 0) return;                                       // never for a row of the step
    if (u < heads + kv_heads) {                                 // a key head
        const int g = u - heads;
        x += heads * D + g * D;
        float scale = 1.0f;
        if (qk_norm) {
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(x[c], x[c], ss);
            scale = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        T* o = k_pages + (((size_t)page * kv_heads + g) * CML_PAGE + pos % CML_PAGE) * D;
        for (int c = lane; c < D; c += 32) o[c] = from_f32<T>(qk_norm ? x[c] * scale * to_f32(k_w[c]) : x[c]);
    } else {                                                    // a value head
        const int g = u - heads - kv_heads;
        x += (heads + kv_heads) * D + g * Dv;
        T* o = v_pages + (((size_t)page * kv_heads + g) * CML_PAGE + pos % CML_PAGE) * Dv;
        for (int c = lane; c < Dv; c += 32) o[c] = from_f32<T>(x[c]);
    }
}

extern "C" int cml_qk_norm_kv_write(const float* proj, long ld, const void* q_w, const void* k_w, int w_dtype, int qk_norm,
                                    float eps, const int* row_seq, const int* row_pos, const int* table, int max_blocks,
                                    void* q_out, void* k_pages, void* v_pages, int dtype, int rows, int heads, int kv_heads,
                                    int D, int Dv, void* stream) {
    if (rows <= 0) return 0;
    const long warps = (long)rows * (heads + 2 * kv_heads);
    dim3 grid((unsigned)((warps + 3) / 4));
    cudaStream_t s = (cudaStream_t)stream;
#define QK_CASE(T_, TW_, D_, DW_)                                                                                          \
    if (dtype == D_ && w_dtype == DW_) {                                                                                   \
        launch_pdl(qk_norm_kv_write_kernel<T_, TW_>, grid, dim3(128), 0, s, proj, ld, (const TW_*)q_w, (const TW_*)k_w, qk_norm, \
                   eps, row_seq, row_pos, table, max_blocks, (T_*)q_out, (T_*)k_pages, (T_*)v_pages, rows, heads, kv_heads, D, \
                   Dv);                                                                                                    \
        return cml_launch_status();                                                                                        \
    }
    QK_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    QK_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    QK_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
    QK_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
#undef QK_CASE
    return CML_ERR_BAD_DTYPE;
}

// q [rows, heads x D]; out [rows, heads x Dv] = softmax(...) V, times sigmoid(gate) where
// gate (float [rows, ldg], at column gate_col) is given. window <= 0: all keys. r1, r2 float
// [heads] or null (no penalty). Dynamic shared memory: D floats per warp for the query.
#define AW_WARPS 4
#define AW_MAX_VREGS 8        // value columns per lane: Dv <= 256

template <typename T>
__global__ void window_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                        const int* __restrict__ table, int max_blocks, const int* __restrict__ row_seq,
                                        const int* __restrict__ row_pos, const float* __restrict__ r1,
                                        const float* __restrict__ r2, const float* __restrict__ gate, long ldg, int gate_col,
                                        T* __restrict__ out, int rows, int heads, int kv_heads, int D, int Dv, int window,
                                        float scale) {
    extern __shared__ float q_sh[];
    pdl_wait();
    pdl_launch_dependents();
    const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * AW_WARPS + warp_in_block;
    if (item >= rows * heads) return;
    const int r = item / heads, hd = item % heads, g = hd / (heads / kv_heads);
    float* qs = q_sh + warp_in_block * D;
    for (int c = lane; c < D; c += 32) qs[c] = to_f32(q[((size_t)r * heads + hd) * D + c]);
    __syncwarp();
    const int i = row_pos[r];
    const int lo = window > 0 ? max(0, i - window + 1) : 0;
    const int* tb = table + (size_t)row_seq[r] * max_blocks;
    const float p1 = r1 ? r1[hd] : 0.f, p2 = r2 ? r2[hd] : 0.f;
    float m = -INFINITY, l = 0.f;
    float acc[AW_MAX_VREGS];
#pragma unroll
    for (int e = 0; e < AW_MAX_VREGS; ++e) acc[e] = 0.f;
    for (int j0 = lo; j0 <= i; j0 += 32) {
        const int j = j0 + lane;
        float sc = -INFINITY;
        int page = -1;
        if (j <= i) {
            page = tb[j / CML_PAGE];
            if (page >= 0) {
                const T* kr = k_pages + (((size_t)page * kv_heads + g) * CML_PAGE + j % CML_PAGE) * D;
                float dot = 0.f;
                for (int c = 0; c < D; ++c) dot = fmaf(qs[c], to_f32(kr[c]), dot);
                sc = dot * scale;
                if (r1) sc -= p1 * log1pf(p2 * (float)(i - j));
            }
        }
        const float m_new = fmaxf(m, warp_max(sc));               // the row's own key is always there: finite
        const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
        const float fix = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * fix + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int e = 0; e < AW_MAX_VREGS; ++e) acc[e] *= fix;
        const int nk = min(32, i - j0 + 1);
        for (int t = 0; t < nk; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const int pg = __shfl_sync(0xffffffffu, page, t);
            if (pg < 0) continue;
            const T* vr = v_pages + (((size_t)pg * kv_heads + g) * CML_PAGE + (j0 + t) % CML_PAGE) * Dv;
#pragma unroll
            for (int e = 0; e < AW_MAX_VREGS; ++e) {
                const int c = lane + 32 * e;
                if (c < Dv) acc[e] = fmaf(pt, to_f32(vr[c]), acc[e]);
            }
        }
    }
    const float inv = 1.0f / l;
    T* o = out + ((size_t)r * heads + hd) * Dv;
    const float* gt = gate ? gate + (size_t)r * ldg + gate_col + hd * Dv : nullptr;
#pragma unroll
    for (int e = 0; e < AW_MAX_VREGS; ++e) {
        const int c = lane + 32 * e;
        if (c < Dv) o[c] = from_f32<T>(acc[e] * inv * (gt ? sigmoid_w(gt[c]) : 1.0f));
    }
}

extern "C" int cml_window_attention(const void* q, const void* k_pages, const void* v_pages, int dtype, const int* table,
                                    int max_blocks, const int* row_seq, const int* row_pos, const float* r1, const float* r2,
                                    const float* gate, long ldg, int gate_col, void* out, int rows, int heads, int kv_heads,
                                    int D, int Dv, int window, float scale, void* stream) {
    if (rows <= 0) return 0;
    if (Dv > 32 * AW_MAX_VREGS || D < 1 || heads % kv_heads) return CML_ERR_BAD_SIZE;
    const long items = (long)rows * heads;
    dim3 grid((unsigned)((items + AW_WARPS - 1) / AW_WARPS));
    const size_t smem = (size_t)AW_WARPS * D * sizeof(float);
    if (smem > 48 * 1024) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(window_attention_kernel<float>, grid, dim3(32 * AW_WARPS), smem, s, (const float*)q, (const float*)k_pages,
                   (const float*)v_pages, table, max_blocks, row_seq, row_pos, r1, r2, gate, ldg, gate_col, (float*)out, rows,
                   heads, kv_heads, D, Dv, window, scale);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(window_attention_kernel<bf16>, grid, dim3(32 * AW_WARPS), smem, s, (const bf16*)q, (const bf16*)k_pages,
                   (const bf16*)v_pages, table, max_blocks, row_seq, row_pos, r1, r2, gate, ldg, gate_col, (bf16*)out, rows,
                   heads, kv_heads, D, Dv, window, scale);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
