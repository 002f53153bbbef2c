// Softmax attention over a sliding window of the paged cache, without rotation, for mixers
// whose keys and values may differ in size: per-head RMS norm of q and k, a penalty on the
// distance between query and key, an output gate.
//
//   score(i, j) = (q_i . k_j) scale - r1[head] ln(1 + r2[head] (i - j)),   0 <= i - j < window
//
// Besides the window, a query may be held to the keys of its own block of `chunk` positions (blocks
// counted from position 0 of the sequence); the softmax denominator may hold one more term
// exp(sink[head]) that has no key and no value; the gate may be one number per head. A second
// preparing kernel normalises q and k over their whole projections (all heads at once) and rotates
// pairs of channels by the position (pairs of neighbours, or of the two halves of the rotated part).
//
// Two kernels. The first normalises q and k (weight per channel, shared by the heads), keeps
// q in the compute type and writes k and v into their pages. The second gives a block to
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

// The same job for mixers that rotate: proj [rows, ld] float holds q, k, v as above. norm_mode 0: q and k as
// they are; 1: RMS norm per head, weights of D channels shared by the heads; 2: RMS norm over the whole q
// projection (heads x D channels at once) and the whole k projection, weights of those sizes. Then the first
// rot_dim channels of every q and k head are rotated by angle = position * inv_freq[i] (float), pairing 1:
// channels (2i, 2i + 1); pairing 0: channels (i, i + rot_dim / 2). One block per row. proj may come as split sums
// (n_splits matrices split_stride apart, added here in split order); the row is staged in shared memory. `extra`
// more columns behind v (the logits of an output gate) are copied, summed, to extra_out [rows, extra].
template <typename T, typename TW>
__global__ void __launch_bounds__(1024) qkv_prepare_kernel(const float* __restrict__ proj, long ld, int n_splits, long split_stride,
                                   int extra, float* __restrict__ extra_out, const TW* __restrict__ q_w,
                                   const TW* __restrict__ k_w, int norm_mode, float eps, const float* __restrict__ inv_freq,
                                   int rot_dim, int pairing, const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                   const int* __restrict__ table, int max_blocks, T* __restrict__ q_out, T* __restrict__ k_pages,
                                   T* __restrict__ v_pages, int heads, int kv_heads, int D, int Dv) {
    __shared__ float red[33];
    __shared__ float2 turn[128];                                // (cosine, sine) of the row's angles, shared by all heads
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float x[];                 // the row: q, k, v and the extra columns
    const int r = blockIdx.x;
    const int qw = heads * D, kw = kv_heads * D, vw = kv_heads * Dv;
    {
        const float* src = proj + (size_t)r * ld;
        const int total = qw + kw + vw + extra;
        for (int c = threadIdx.x; c < total; c += blockDim.x) {
            // eight splits at a time: the loads are unconditional (of a valid place) and all in flight before the
            // first add; the adds stay in split order
            float v = src[c];
            for (int s0 = 1; s0 < n_splits; s0 += 8) {
                float t[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) t[k] = src[(size_t)min(s0 + k, n_splits - 1) * split_stride + c];
#pragma unroll
                for (int k = 0; k < 8; ++k) v += s0 + k < n_splits ? t[k] : 0.f;
            }
            x[c] = v;
            if (c >= total - extra) extra_out[(size_t)r * extra + (c - (total - extra))] = v;
        }
    }
    const int pos = row_pos[r];
    for (int i = threadIdx.x; i < rot_dim / 2; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        turn[i] = make_float2(cs, sn);
    }
    __syncthreads();
    const int page = table[(size_t)row_seq[r] * max_blocks + pos / CML_PAGE];
    float q_scale = 1.0f, k_scale = 1.0f;
    if (norm_mode == 2) {
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < qw; c += blockDim.x) sq = fmaf(x[c], x[c], sq);
        for (int c = threadIdx.x; c < kw; c += blockDim.x) sk = fmaf(x[qw + c], x[qw + c], sk);
        q_scale = 1.0f / sqrtf(block_sum(sq, red) / (float)qw + eps);
        __syncthreads();
        k_scale = 1.0f / sqrtf(block_sum(sk, red) / (float)kw + eps);
        __syncthreads();
    }
    float* head_scale = x + qw + kw + vw + extra;               // norm per head: one scale per q and k head
    if (norm_mode == 1) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
        for (int u = warp; u < heads + kv_heads; u += nwarps) {
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(x[u * D + c], x[u * D + c], ss);
            ss = warp_sum(ss);
            if (lane == 0) head_scale[u] = 1.0f / sqrtf(ss / (float)D + eps);
        }
        __syncthreads();
    }
    const int half = rot_dim / 2;
    // Channel c of the q | k stretch after norm and rotation. Its partner in the rotation is its neighbour (pairing 1)
    // or the channel half the rotated part away (pairing 0); the first of a pair becomes u cos - v sin, the second
    // v cos + u sin.
    auto channel = [&](int c) -> float {
        const bool is_q = c < qw;
        const int cc = is_q ? c : c - qw;                       // column within the q or the k projection
        const int u = c / D, d = c - u * D;                     // head among q and k heads, channel within it
        const TW* w = is_q ? q_w : k_w;
        const float sc = norm_mode == 2 ? (is_q ? q_scale : k_scale) : norm_mode == 1 ? head_scale[u] : 1.0f;
        const int wi = norm_mode == 2 ? cc : d;
        const float a = norm_mode ? x[c] * sc * to_f32(w[wi]) : x[c];
        if (d >= rot_dim) return a;
        const bool first = pairing ? !(d & 1) : d < half;
        const int off = pairing ? (first ? 1 : -1) : (first ? half : -half);
        const float b = norm_mode ? x[c + off] * sc * to_f32(w[wi + off]) : x[c + off];
        const float2 t = turn[pairing ? d >> 1 : (first ? d : d - half)];
        return first ? a * t.x - b * t.y : a * t.x + b * t.y;
    };
    T* k_row = page >= 0 ? k_pages + ((size_t)page * kv_heads * CML_PAGE + pos % CML_PAGE) * D : nullptr;
    if ((D & 1) == 0) {                                          // two neighbouring channels a thread: 4-byte stores of bfloat16
        for (int c = threadIdx.x * 2; c < qw + kw; c += blockDim.x * 2) {
            const float o0 = channel(c), o1 = channel(c + 1);
            T* o;
            if (c < qw) o = q_out + (size_t)r * qw + c;
            else {
                if (k_row == nullptr) continue;
                const int g = (c - qw) / D;
                o = k_row + (size_t)g * CML_PAGE * D + (c - qw - g * D);
            }
            o[0] = from_f32<T>(o0);
            o[1] = from_f32<T>(o1);
        }
    } else {
        for (int c = threadIdx.x; c < qw + kw; c += blockDim.x) {
            const float o0 = channel(c);
            if (c < qw) q_out[(size_t)r * qw + c] = from_f32<T>(o0);
            else if (k_row != nullptr) {
                const int g = (c - qw) / D;
                k_row[(size_t)g * CML_PAGE * D + (c - qw - g * D)] = from_f32<T>(o0);
            }
        }
    }
    if (page >= 0) {
        for (int c = threadIdx.x; c < vw; c += blockDim.x) {
            const int g = c / Dv, e = c - g * Dv;
            v_pages[(((size_t)page * kv_heads + g) * CML_PAGE + pos % CML_PAGE) * Dv + e] = from_f32<T>(x[qw + kw + c]);
        }
    }
}

extern "C" int cml_qkv_prepare(const float* proj, long ld, int n_splits, long split_stride, int extra, float* extra_out, const void* q_w, const void* k_w, int w_dtype, int norm_mode, float eps,
                               const float* inv_freq, int rot_dim, int pairing, const int* row_seq, const int* row_pos,
                               const int* table, int max_blocks, void* q_out, void* k_pages, void* v_pages, int dtype, int rows,
                               int heads, int kv_heads, int D, int Dv, void* stream) {
    if (rows <= 0) return 0;
    if (rot_dim < 0 || rot_dim > D || rot_dim > 256 || (rot_dim & 1) || norm_mode < 0 || norm_mode > 2) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (n_splits < 1 || extra < 0) return CML_ERR_BAD_SIZE;
    const size_t smem = (size_t)(heads * D + kv_heads * (D + Dv) + extra + heads + kv_heads) * sizeof(float);
    if (smem > 200 * 1024) return CML_ERR_BAD_SIZE;
#define QP_CASE(T_, TW_, D_, DW_)                                                                                          \
    if (dtype == D_ && w_dtype == DW_) {                                                                                   \
        if (smem > 48 * 1024 && cml_allow_smem<qkv_prepare_kernel<T_, TW_>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE; \
        launch_pdl(qkv_prepare_kernel<T_, TW_>, dim3(rows), dim3(rows <= 128 ? 1024 : 256), smem, s, proj, ld, n_splits, split_stride, extra,   \
                   extra_out, (const TW_*)q_w, (const TW_*)k_w,                                                            \
                   norm_mode, eps, inv_freq, rot_dim, pairing, row_seq, row_pos, table, max_blocks, (T_*)q_out,            \
                   (T_*)k_pages, (T_*)v_pages, heads, kv_heads, D, Dv);                                                    \
        return cml_launch_status();                                                                                        \
    }
    QP_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    QP_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    QP_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
    QP_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
#undef QP_CASE
    return CML_ERR_BAD_DTYPE;
}

// q [rows, heads x D]; out [rows, heads x Dv] = softmax(...) V, times sigmoid(gate) where
// gate (float [rows, ldg], at column gate_col) is given. window <= 0: all keys. r1, r2 float
// [heads] or null (no penalty).
//
// A block of NW warps owns one (row, head). The visible keys, oldest first, are dealt to the
// warps in runs of whole rounds of 32 (how many depends on the row's position and the window
// alone, not on how the prompt was cut); in a round a lane takes one key for the score (the key
// row read in 16-byte pieces where its size allows) and then columns of the values; each warp
// keeps an online softmax of its run, and the runs are merged in warp order at the end.
// Dynamic shared memory: the query (D floats), then per warp its maximum, its sum and Dv sums.
#define AW_MAX_VREGS 8        // value columns per lane at most: Dv <= 256

template <typename T> struct Piece;                 // 16 bytes of a key row as floats
template <> struct Piece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ uint4 raw(const float* p) { return *reinterpret_cast<const uint4*>(p); }
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ void load(const float* p, float* f) { unpack(raw(p), f); }
};
template <> struct Piece<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ uint4 raw(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
    static __device__ __forceinline__ void load(const bf16* p, float* f) { unpack(raw(p), f); }
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <typename T, int NV>              // NV: value columns per lane, Dv <= 32 * NV
__global__ void __launch_bounds__(512, 1) window_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                        const int* __restrict__ table, int max_blocks, const int* __restrict__ row_seq,
                                        const int* __restrict__ row_pos, const float* __restrict__ r1,
                                        const float* __restrict__ r2, const float* __restrict__ gate, long ldg, int gate_col,
                                        T* __restrict__ out, int heads, int kv_heads, int D, int Dv, int window, float scale,
                                        int chunk, const float* __restrict__ sink, int gate_per_head) {
    extern __shared__ __align__(16) float aw_sh[];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int r = blockIdx.x / heads, hd = blockIdx.x % heads, g = hd / (heads / kv_heads);
    float* qs = aw_sh;
    float* part = aw_sh + ((D + 3) & ~3) + warp * (Dv + 2);
    // what the first round needs besides the query is asked for before the query is staged
    const int i = row_pos[r];
    int lo = window > 0 ? max(0, i - window + 1) : 0;
    if (chunk > 0) lo = max(lo, i - i % chunk);             // the first position of the row's own block
    const int rounds = (i - lo) / 32 + 1;
    const int per_warp = (rounds + nw - 1) / nw;
    const int j_first = lo + 32 * warp * per_warp, j_end = min(i + 1, j_first + 32 * per_warp);
    const int* tb = table + (size_t)row_seq[r] * max_blocks;
    int page_first = -1;
    if (j_first + lane < j_end) page_first = tb[(j_first + lane) / CML_PAGE];
    for (int c = threadIdx.x; c < D; c += blockDim.x) qs[c] = to_f32(q[((size_t)r * heads + hd) * D + c]);
    __syncthreads();
    const float p1 = r1 ? r1[hd] : 0.f, p2 = r2 ? r2[hd] : 0.f;
    const bool pieces = (D % Piece<T>::N) == 0;              // a key row is a whole number of 16-byte pieces
    float m = -INFINITY, l = 0.f;
    float acc[NV];
#pragma unroll
    for (int e = 0; e < NV; ++e) acc[e] = 0.f;
    constexpr int PN = Piece<T>::N;
    constexpr int KB = NV >= 8 ? 8 : 16;                     // keys whose values are in flight together
    for (int j0 = j_first; j0 < j_end; j0 += 32) {
        const int j = j0 + lane;
        float sc = -INFINITY;
        int page = -1;
        if (j < j_end) {
            page = j0 == j_first ? page_first : tb[j / CML_PAGE];
            if (page >= 0) {
                const T* kr = k_pages + (((size_t)page * kv_heads + g) * CML_PAGE + j % CML_PAGE) * D;
                float dot = 0.f;
                if (pieces) {
                    // sixteen 16-byte pieces of the key row in flight (a whole row of 128 bfloat16), then their
                    // products; what is left in fours and singly. The sum runs over the channels in order either way.
                    int c = 0;
                    for (; c + 16 * PN <= D; c += 16 * PN) {
                        uint4 raw[16];
#pragma unroll
                        for (int u = 0; u < 16; ++u) raw[u] = Piece<T>::raw(kr + c + u * PN);
#pragma unroll
                        for (int u = 0; u < 16; ++u) {
                            float kf[PN];
                            Piece<T>::unpack(raw[u], kf);
#pragma unroll
                            for (int x = 0; x < PN; ++x) dot = fmaf(qs[c + u * PN + x], kf[x], dot);
                        }
                    }
                    for (; c + 4 * PN <= D; c += 4 * PN) {
                        uint4 raw[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) raw[u] = Piece<T>::raw(kr + c + u * PN);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            float kf[PN];
                            Piece<T>::unpack(raw[u], kf);
#pragma unroll
                            for (int x = 0; x < PN; ++x) dot = fmaf(qs[c + u * PN + x], kf[x], dot);
                        }
                    }
                    for (; c < D; c += PN) {
                        float kf[PN];
                        Piece<T>::load(kr + c, kf);
#pragma unroll
                        for (int x = 0; x < PN; ++x) dot = fmaf(qs[c + x], kf[x], dot);
                    }
                } else {
                    for (int c = 0; c < D; ++c) dot = fmaf(qs[c], to_f32(kr[c]), dot);
                }
                sc = dot * scale;
                if (r1) sc -= p1 * log1pf(p2 * (float)(i - j));
            }
        }
        const float m_new = fmaxf(m, warp_max(sc));
        const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
        const float fix = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * fix + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int e = 0; e < NV; ++e) acc[e] *= fix;
        const int nk = min(32, j_end - j0);
        // KB keys at a time: their weights and pages by shuffles first, then all their value loads (each
        // unconditional, of a valid row: a key that does not count has weight zero), then the sums in key order
        for (int t0 = 0; t0 < nk; t0 += KB) {
            float pt[KB];
            const T* vr[KB];
#pragma unroll
            for (int u = 0; u < KB; ++u) {
                const int t = min(t0 + u, nk - 1);
                const int pg = __shfl_sync(0xffffffffu, page, t);
                const float pp = __shfl_sync(0xffffffffu, p, t);
                pt[u] = (t0 + u < nk && pg >= 0) ? pp : 0.f;
                vr[u] = v_pages + (((size_t)max(pg, 0) * kv_heads + g) * CML_PAGE + (j0 + t) % CML_PAGE) * Dv;
            }
            float vv[KB][NV];
#pragma unroll
            for (int u = 0; u < KB; ++u)
#pragma unroll
                for (int e = 0; e < NV; ++e) {
                    const int c = lane + 32 * e;
                    vv[u][e] = to_f32(vr[u][c < Dv ? c : 0]);
                }
#pragma unroll
            for (int u = 0; u < KB; ++u)
#pragma unroll
                for (int e = 0; e < NV; ++e) acc[e] = fmaf(pt[u], vv[u][e], acc[e]);
        }
    }
    if (lane == 0) { part[0] = m; part[1] = l; }
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int c = lane + 32 * e;
        if (c < Dv) part[2 + c] = acc[e];
    }
    __syncthreads();
    // the runs merged in warp order (warp 0 always has the oldest visible key, so the maximum is finite)
    const float* parts = aw_sh + ((D + 3) & ~3);
    float top = -INFINITY;
    for (int w = 0; w < nw; ++w) top = fmaxf(top, parts[w * (Dv + 2)]);
    const float snk = sink ? sink[hd] : -INFINITY;              // one more term of the denominator, without a value
    top = fmaxf(top, snk);
    float total = 0.f;
    for (int w = 0; w < nw; ++w) {
        const float mw = parts[w * (Dv + 2)];
        if (mw != -INFINITY) total += parts[w * (Dv + 2) + 1] * expf(mw - top);
    }
    if (sink) total += expf(snk - top);
    const float inv = 1.0f / total;
    T* o = out + ((size_t)r * heads + hd) * Dv;
    const float* gt = gate ? gate + (size_t)r * ldg + gate_col + (gate_per_head ? hd : hd * Dv) : nullptr;
    const int gstep = gate_per_head ? 0 : 1;
    for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
        float sum = 0.f;
        for (int w = 0; w < nw; ++w) {
            const float mw = parts[w * (Dv + 2)];
            if (mw != -INFINITY) sum += parts[w * (Dv + 2) + 2 + c] * expf(mw - top);
        }
        o[c] = from_f32<T>(sum * inv * (gt ? sigmoid_w(gt[c * gstep]) : 1.0f));
    }
}

extern "C" int cml_window_attention(const void* q, const void* k_pages, const void* v_pages, int dtype, const int* table,
                                    int max_blocks, const int* row_seq, const int* row_pos, const float* r1, const float* r2,
                                    const float* gate, long ldg, int gate_col, void* out, int rows, int heads, int kv_heads,
                                    int D, int Dv, int window, float scale, int chunk, const float* sink, int gate_per_head,
                                    void* stream) {
    if (rows <= 0) return 0;
    if (Dv > 32 * AW_MAX_VREGS || D < 1 || heads % kv_heads) return CML_ERR_BAD_SIZE;
    // warps per (row, head): one per round of 32 keys of the window, at most 16 (8 without a window); fixed by
    // the window alone, so a row's sums do not depend on the step it came in
    // (or by the block of positions, whichever lets a query see fewer keys)
    int span = window > 0 ? window : 0;
    if (chunk > 0 && (span == 0 || chunk < span)) span = chunk;
    const int nw = span > 0 ? ((span + 31) / 32 < 16 ? (span + 31) / 32 : 16) : 8;
    dim3 grid((unsigned)((long)rows * heads));
    const size_t smem = (size_t)(((D + 3) & ~3) + nw * (Dv + 2)) * sizeof(float);
    if (smem > 48 * 1024 || (long)rows * heads > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
#define AW_CASE(T_, NV_)                                                                                                    \
    launch_pdl(window_attention_kernel<T_, NV_>, grid, dim3(32 * nw), smem, s, (const T_*)q, (const T_*)k_pages, (const T_*)v_pages, \
               table, max_blocks, row_seq, row_pos, r1, r2, gate, ldg, gate_col, (T_*)out, heads, kv_heads, D, Dv, window, scale, \
               chunk, sink, gate_per_head)
#define AW_SIZES(T_)                                                                                                        \
    if (Dv <= 32) AW_CASE(T_, 1); else if (Dv <= 64) AW_CASE(T_, 2); else if (Dv <= 128) AW_CASE(T_, 4); else AW_CASE(T_, 8)
    if (dtype == CML_DTYPE_F32) { AW_SIZES(float); }
    else if (dtype == CML_DTYPE_BF16) { AW_SIZES(bf16); }
    else return CML_ERR_BAD_DTYPE;
#undef AW_SIZES
#undef AW_CASE
    return cml_launch_status();
}
