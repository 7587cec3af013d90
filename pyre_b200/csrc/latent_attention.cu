// Attention over a cache of LATENT rows: per token the paged cache holds one row [c | r] shared by all heads,
// c the low-rank latent (`rank` entries, RMS-normed) from which every head's keys and values are linear maps,
// r a rotated key part (`rope` entries).  The kernels here work in the absorbed form: a head's key map is applied
// to its QUERY (q~ = U_k^T q, a product done elsewhere), so that the score of head h for key j is
// (q~_h . c_j + qr_h . r_j) * scale and the head's output before its value map is sum_j p_j c_j.  Keys and
// values are never expanded per head; one cache row serves all heads of a token as key and as value.
//
//   latent_prepare   norms of the two down-projections, rotation of the shared key part, the paged write
//   latent_rotate_q  rotation of the queries' rotated part into the absorbed query rows
//   latent_attention_exact   fp32 arithmetic, any sizes, bit-identical under cutting and batching
//
// Rotation (neighbouring pairs): (u, v) = (x[2i], x[2i + 1]) -> (u cos a - v sin a, v cos a + u sin a), i < rot / 2,
// with cos/sin of the token's angles from a table [T, rot / 2]; entries from `rot` on pass unchanged.
// `dtype`: type of activations and cache (0 = float32, 1 = bfloat16); all arithmetic is fp32.
#include "common.cuh"

template <typename T>
__device__ __forceinline__ float proj_at(const T* proj, const float* parts, int n_parts, long long part_stride, size_t at) {
    if (parts) {
        float acc = parts[at];
        for (int s = 1; s < n_parts; ++s) acc += parts[(size_t)s * part_stride + at];
        return acc;
    }
    return to_f32<T>(proj[at]);
}

// ---------------------------------------------------------------------------
// proj [T, W] (activation dtype, or fp32 partial sums): columns [q_col, q_col + q_rank) the query latent,
// [c_col, c_col + rank) the key/value latent, [c_col + rank, c_col + rank + rope) the shared key part.
//   cq_out[t]      = rmsnorm(query latent) * wq            [T, q_rank]   (q_rank = 0: none)
//   cache[slot[t]] = [ rmsnorm(latent) * wc | rotate(key part) ]          rows of `row` >= rank + rope entries
// One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void latent_prepare_kernel(const T* proj, const float* parts, int n_parts, long long part_stride, int W,
                                      int q_col, int q_rank, int c_col, int rank, int rope, int rot, const float* wq,
                                      const float* wc, float eps, const float* cos_t, const float* sin_t, T* cq_out,
                                      T* cache, const int* slot_mapping, int row, long long n_pages, int page_size,
                                      int* err_flag) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const size_t base = (size_t)t * W;
    if (q_rank > 0) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = proj_at<T>(proj, parts, n_parts, part_stride, base + q_col + i);
            ss = fmaf(v, v, ss);
        }
        const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = proj_at<T>(proj, parts, n_parts, part_stride, base + q_col + i);
            cq_out[(size_t)t * q_rank + i] = from_f32<T>(__fmul_rn(__fmul_rn(v, rstd), wq[i]));
        }
    }
    const int slot = cache ? pyre_checked_slot(slot_mapping[t], n_pages, page_size, err_flag) : -1;
    if (slot < 0) return;   // the whole block
    T* dst = cache + (size_t)slot * row;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = proj_at<T>(proj, parts, n_parts, part_stride, base + c_col + i);
        ss = fmaf(v, v, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = proj_at<T>(proj, parts, n_parts, part_stride, base + c_col + i);
        dst[i] = from_f32<T>(__fmul_rn(__fmul_rn(v, rstd), wc[i]));
    }
    const int half = rot / 2;
    for (int i = threadIdx.x; i < rope; i += blockDim.x) {
        const float v = proj_at<T>(proj, parts, n_parts, part_stride, base + c_col + rank + i);
        float o = v;
        if (i < rot) {
            const float other = proj_at<T>(proj, parts, n_parts, part_stride, base + c_col + rank + (i ^ 1));
            const float c = cos_t[(size_t)t * half + (i >> 1)], s = sin_t[(size_t)t * half + (i >> 1)];
            o = (i & 1) ? fmaf(v, c, __fmul_rn(other, s)) : fmaf(v, c, -__fmul_rn(other, s));
        }
        dst[rank + i] = from_f32<T>(o);
    }
    for (int i = rank + rope + threadIdx.x; i < row; i += blockDim.x) dst[i] = from_f32<T>(0.f);
}

PYRE_API int pyre_latent_prepare(const void* proj, const float* parts, int n_parts, long long part_stride, int W, int q_col,
                                 int q_rank, int c_col, int rank, int rope, int rot, const float* wq, const float* wc,
                                 float eps, const float* cos_t, const float* sin_t, void* cq_out, void* cache,
                                 const int* slot_mapping, int n_tokens, int row, long long n_pages, int page_size,
                                 int dtype, int* err_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if ((proj == nullptr) == (parts == nullptr) || rank <= 0 || rope < 0 || rot < 0 || rot > rope || rot % 2 ||
        row < rank + rope || (q_rank > 0 && (!wq || !cq_out)) || !wc || (cache && !slot_mapping) ||
        (rot > 0 && (!cos_t || !sin_t)))
        return PYRE_ERR_BAD_ARG;
    const int threads = 128;
    if (dtype == PYRE_BF16)
        pyre_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)proj, parts,
                    n_parts, part_stride, W, q_col, q_rank, c_col, rank, rope, rot, wq, wc, eps, cos_t, sin_t,
                    (__nv_bfloat16*)cq_out, (__nv_bfloat16*)cache, slot_mapping, row, n_pages, page_size, err_flag);
    else if (dtype == PYRE_F32)
        pyre_launch(latent_prepare_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)proj, parts, n_parts,
                    part_stride, W, q_col, q_rank, c_col, rank, rope, rot, wq, wc, eps, cos_t, sin_t, (float*)cq_out,
                    (float*)cache, slot_mapping, row, n_pages, page_size, err_flag);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// q [T, nh, dq + rope] (a head's plain part, then its rotated part) -> qa[t, h, rank + i] = rotate(q[t, h, dq + i]),
// i < rope, and zeros from rank + rope to `row`: the tail of the absorbed query rows [T, nh, row], whose first
// `rank` entries a product writes.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void latent_rotate_q_kernel(const T* q, T* qa, const float* cos_t, const float* sin_t, int n_tokens, int nh,
                                       int dq, int rope, int rot, int rank, int row) {
    pdl_trigger();
    pdl_wait();
    const int tail = row - rank;
    const size_t total = (size_t)n_tokens * nh * tail;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int half = rot / 2;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t th = idx / tail;
        const int i = (int)(idx - th * tail);
        const int t = (int)(th / nh);
        float o = 0.f;
        if (i < rope) {
            const T* src = q + th * (size_t)(dq + rope) + dq;
            const float v = to_f32<T>(src[i]);
            o = v;
            if (i < rot) {
                const float other = to_f32<T>(src[i ^ 1]);
                const float c = cos_t[(size_t)t * half + (i >> 1)], s = sin_t[(size_t)t * half + (i >> 1)];
                o = (i & 1) ? fmaf(v, c, __fmul_rn(other, s)) : fmaf(v, c, -__fmul_rn(other, s));
            }
        }
        qa[th * (size_t)row + rank + i] = from_f32<T>(o);
    }
}

PYRE_API int pyre_latent_rotate_q(const void* q, void* qa, const float* cos_t, const float* sin_t, int n_tokens, int nh, int dq,
                                  int rope, int rot, int rank, int row, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || nh <= 0 || row <= rank) return 0;
    if (rot < 0 || rot > rope || rot % 2 || row < rank + rope || (rot > 0 && (!cos_t || !sin_t))) return PYRE_ERR_BAD_ARG;
    const long long total = (long long)n_tokens * nh * (row - rank);
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll(total, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(latent_rotate_q_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)qa,
                    cos_t, sin_t, n_tokens, nh, dq, rope, rot, rank, row);
    else if (dtype == PYRE_F32)
        pyre_launch(latent_rotate_q_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)q, (float*)qa, cos_t, sin_t,
                    n_tokens, nh, dq, rope, rot, rank, row);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// The exact kernel.  One warp owns one (query token, head) and walks the cached rows of the token's sequence
// in chunks of 32 aligned to position 0, from the start of its window to its own position, with an online
// softmax.  A lane scores one row (the dot product over all `kd` = rank + rope key entries of the row), then the
// warp adds the 32 rows' first `rank` entries weighted by their probabilities.  Every sum has a fixed order that
// depends on the token's own keys only.
//   qa [T, nh, row]: absorbed queries; cache: one layer [page][page_size][row]; out [T, nh, rank]
// ---------------------------------------------------------------------------
constexpr int LATENT_MAX_RANK = 512;

template <typename T>
__global__ void latent_attention_exact_kernel(const T* qa, const T* cache, T* out, const int* block_table, int bt_stride,
                                              const int* seq_of_token, const int* positions, int n_tokens, int nh, int rank,
                                              int kd, int row, int page_size, int window, float scale, long long n_pages,
                                              int* err_flag) {
    extern __shared__ float q_smem[];   // [warps][kd]
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps + warp;
    if (item >= (long long)n_tokens * nh) return;
    const int t = (int)(item / nh);
    const int seq = seq_of_token[t];
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_table + (size_t)seq * bt_stride;
    float* qs = q_smem + warp * kd;
    const T* qrow = qa + (size_t)item * row;
    for (int d = lane; d < kd; d += 32) qs[d] = to_f32<T>(qrow[d]);
    __syncwarp();

    constexpr int OWN = LATENT_MAX_RANK / 32;
    const int n_own = (rank + 31) / 32;
    float acc[OWN];
#pragma unroll
    for (int i = 0; i < OWN; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const bool vec8 = (row % 8 == 0) && (kd % 8 == 0);

    for (int c = (lo / 32) * 32; c <= pos; c += 32) {
        const int j = c + lane;
        const bool valid = j >= lo && j <= pos;
        float score = -INFINITY;
        long long vrow = -1;
        if (valid) {
            const int page = pyre_checked_page(table[j / page_size], n_pages, err_flag);
            vrow = (long long)page * page_size + j % page_size;
            const T* kp = cache + (size_t)vrow * row;
            float dot[4] = {0.f, 0.f, 0.f, 0.f};
            if (vec8) {
                for (int d = 0; d < kd; d += 8) {
                    Vec<T, 8> kv = load_vec<T, 8>(kp + d);
#pragma unroll
                    for (int e = 0; e < 8; ++e) dot[e & 3] = fmaf(qs[d + e], to_f32<T>(kv.v[e]), dot[e & 3]);
                }
            } else {
                for (int d = 0; d < kd; ++d) dot[d & 3] = fmaf(qs[d], to_f32<T>(kp[d]), dot[d & 3]);
            }
            score = ((dot[0] + dot[1]) + (dot[2] + dot[3])) * scale;
        }
        const float m_new = fmaxf(m, warp_max(score));
        const float p = valid ? expf(score - m_new) : 0.f;
        const float alpha = expf(m - m_new);
        l = l * alpha + warp_sum(p);
        float part[OWN];
#pragma unroll
        for (int i = 0; i < OWN; ++i) part[i] = 0.f;
        const int n_keys = min(32, pos - c + 1);
        for (int jj = 0; jj < n_keys; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long vr = __shfl_sync(0xffffffffu, vrow, jj);
            if (vr < 0) continue;   // before the window: the same for the whole warp
            const T* vp = cache + (size_t)vr * row;
#pragma unroll
            for (int i = 0; i < OWN; ++i) {
                const int d = lane + 32 * i;
                if (i < n_own && d < rank) part[i] = fmaf(pj, to_f32<T>(vp[d]), part[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < OWN; ++i) acc[i] = fmaf(acc[i], alpha, part[i]);
        m = m_new;
    }
    const float inv_l = 1.0f / l;
    T* orow = out + (size_t)item * rank;
#pragma unroll
    for (int i = 0; i < OWN; ++i) {
        const int d = lane + 32 * i;
        if (i < n_own && d < rank) orow[d] = from_f32<T>(acc[i] * inv_l);
    }
}

PYRE_API int pyre_latent_attention_exact(const void* qa, const void* cache, void* out, const int* block_table, int bt_stride,
                                         const int* seq_of_token, const int* positions, int n_tokens, int nh, int rank,
                                         int rope, int row, int page_size, int window, float scale, int dtype,
                                         long long n_pages, int* err_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || rope < 0 || row < rank + rope || nh <= 0 || page_size <= 0) return PYRE_ERR_BAD_ARG;
    if (rank > LATENT_MAX_RANK) return PYRE_ERR_UNSUPPORTED;
    const int kd = rank + rope;
    const int warps = 4;
    const long long items = (long long)n_tokens * nh;
    const int blocks = (int)ceil_div_ll(items, warps);
    const size_t smem = (size_t)warps * kd * sizeof(float);
    if (smem > 48 * 1024) return PYRE_ERR_UNSUPPORTED;
    if (dtype == PYRE_F32)
        pyre_launch(latent_attention_exact_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream, (const float*)qa,
                    (const float*)cache, (float*)out, block_table, bt_stride, seq_of_token, positions, n_tokens, nh, rank, kd,
                    row, page_size, window, scale, n_pages, err_flag);
    else if (dtype == PYRE_BF16)
        pyre_launch(latent_attention_exact_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream, (const __nv_bfloat16*)qa,
                    (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, block_table, bt_stride, seq_of_token, positions, n_tokens,
                    nh, rank, kd, row, page_size, window, scale, n_pages, err_flag);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}
