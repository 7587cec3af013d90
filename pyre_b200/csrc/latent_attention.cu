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

// ---------------------------------------------------------------------------
// bfloat16 on the tensor cores (mma.sync m16n8k16, fp32 accumulators), for prompt portions and decoded tokens
// alike.  All heads of a token read the same cached rows, so the heads are stacked on the MMA's rows: a CTA owns 64
// rows = (token, head) pairs of one entry (`hg` heads per token, 64 / hg tokens), four warps of 16 rows.  The keys
// of the tile's window travel through shared memory in tiles of 32 rows (cp.async, two buffers); a cached row is
// the key (all `kd` entries, S = Q K^T) and, by its first `rank` entries, the value (O += P V, the B operand
// fetched with ldmatrix.trans from the same tile).  Softmax online in fp32; P enters the second product as bf16.
// A warp holds 128 output columns of its 16 rows; a latent wider than that takes more warps per row group (up to
// four: 16 warps per CTA), which share the key tiles in shared memory; the warps of a row group then split the
// inner dimension of S = Q K^T among them and exchange their partial scores through shared memory (added in a
// fixed order), so S is computed once.  With `n_splits` > 1 the key tiles of a row tile are shared among that many CTAs, which leave
// unnormalised partial outputs with their maxima and sums in scratch memory for the combining kernel.
//   qa [T, nh, row] absorbed queries (zeros beyond kd); cache [page][page_size][row]; out [T, nh, rank]
//   row % 16 == 0 (the padding of queries and cache rows is zero, so it adds nothing to a score)
// ---------------------------------------------------------------------------
constexpr int LM_ROWS = 64, LM_KT = 32, LM_DV = 128;

__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(512) latent_attention_mma_kernel(
    const __nv_bfloat16* qa, const __nv_bfloat16* cache, __nv_bfloat16* out, float* part_o, float* part_ml,
    const int* block_table, int bt_stride, const int* cu_seqlens, const int* positions, int n_seqs, int nh, int hg, int rank,
    int row, int page_size, int window, float scale_log2, int n_splits, int max_len, long long n_pages, int* err_flag) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    __shared__ int item[3];
    pdl_trigger();
    pdl_wait();
    const int ld = row + 8;                                      // padded row of the shared tiles, in elements
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);          // [64][ld]
    __nv_bfloat16* k_s = q_s + LM_ROWS * ld;                                  // [2][32][ld]
    float* sx = reinterpret_cast<float*>(k_s + 2 * LM_KT * ld);               // [4 row groups][column groups][16][32]: partial scores
    const int n_cg = blockDim.x >> 7;                                         // column groups = warps per row group
    const int tq = LM_ROWS / hg;                                 // tokens of a row tile
    if (threadIdx.x == 0) {
        int tile = blockIdx.x;
        item[0] = -1;
        for (int b = 0; b < n_seqs; ++b) {
            const int n = cu_seqlens[b + 1] - cu_seqlens[b];
            if (max_len > 0 && n > max_len) continue;            // entries that another kernel takes
            const int tiles = (n + tq - 1) / tq;
            if (tile < tiles) {
                item[0] = b;
                item[1] = cu_seqlens[b] + tile * tq;
                item[2] = min(tq, n - tile * tq);
                break;
            }
            tile -= tiles;
        }
    }
    __syncthreads();
    const int seq = item[0];
    if (seq < 0) return;
    const int tok0 = item[1], ntok = item[2];
    const int h0 = blockIdx.y * hg, nhere = min(hg, nh - h0);
    const int lane = threadIdx.x & 31, warp_all = threadIdx.x >> 5;
    const int warp = warp_all & 3, chunk = warp_all >> 2;        // the warp's 16 rows; its 128 output columns
    const int split = blockIdx.z;
    const int c0 = chunk * LM_DV;                                // first output column of this warp
    const int p_first = positions[tok0];
    const int k_hi = p_first + ntok - 1;
    const int k_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    const int k_al = (k_lo / LM_KT) * LM_KT;
    const int tiles_total = (k_hi + 1 - k_al + LM_KT - 1) / LM_KT;
    const int per = (tiles_total + n_splits - 1) / n_splits;
    const int tile_lo = split * per, tile_hi = min(tiles_total, tile_lo + per);
    const int* table = block_table + (size_t)seq * bt_stride;
    const int vecs = row / 8;                                    // 16-byte pieces of a row

    // the queries of the tile's rows
    for (int idx = threadIdx.x; idx < LM_ROWS * vecs; idx += blockDim.x) {
        const int r = idx / vecs, v = idx - r * vecs;
        const int tt = r / hg, hh = r - tt * hg;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (tt < ntok && hh < nhere) val = *reinterpret_cast<const uint4*>(qa + ((size_t)(tok0 + tt) * nh + h0 + hh) * row + v * 8);
        *reinterpret_cast<uint4*>(q_s + r * ld + v * 8) = val;
    }
    // a thread fetches pieces of ONE cached row per tile (blockDim / 32 threads share a row): one look at the block
    // table per thread and tile
    const int tpr = blockDim.x / LM_KT, key_j = threadIdx.x / tpr, key_v = threadIdx.x - key_j * tpr;
    auto load_keys = [&](int buf, int tile) {
        __nv_bfloat16* d = k_s + (size_t)buf * LM_KT * ld + key_j * ld;
        const int pos = k_al + tile * LM_KT + key_j;
        if (pos >= k_lo && pos <= k_hi) {
            const int page = pyre_checked_page(table[pos / page_size], n_pages, err_flag);
            const __nv_bfloat16* src = cache + ((size_t)page * page_size + pos % page_size) * row;
            for (int v = key_v; v < vecs; v += tpr) {
                const uint32_t daddr = (uint32_t)__cvta_generic_to_shared(d + v * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(daddr), "l"(src + v * 8));
            }
        } else {
            for (int v = key_v; v < vecs; v += tpr) *reinterpret_cast<uint4*>(d + v * 8) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;" ::);
    };

    // this thread's two rows: g and g + 8 of the warp's 16
    int p_row[2], lo_row[2];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = warp * 16 + (lane >> 2) + u * 8;
        const int tt = r / hg, hh = r - tt * hg;
        live[u] = tt < ntok && hh < nhere;
        p_row[u] = p_first + tt;
        lo_row[u] = (window > 0 && p_row[u] - window + 1 > 0) ? p_row[u] - window + 1 : 0;
    }
    float o[LM_DV / 8][4];
#pragma unroll
    for (int i = 0; i < LM_DV / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const bool warp_live = warp * 16 < ntok * hg;                // rows beyond the tile's tokens: nothing to compute
    const int nt_live = min(LM_DV, ((rank - c0 + 7) / 8) * 8) / 8;      // 8-column tiles of the output that exist here

    if (tile_lo < tile_hi) load_keys(0, tile_lo);
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int buf = (tile - tile_lo) & 1;
        if (tile + 1 < tile_hi) {
            load_keys(buf ^ 1, tile + 1);
            asm volatile("cp.async.wait_group 1;" ::);
        } else {
            asm volatile("cp.async.wait_group 0;" ::);
        }
        __syncthreads();
        const __nv_bfloat16* kt = k_s + (size_t)buf * LM_KT * ld;
        if (!warp_live) {
            __syncthreads();
            continue;
        }
        float s[LM_KT / 8][4];
#pragma unroll
        for (int i = 0; i < LM_KT / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
        const int ks_per = (row / 16 + n_cg - 1) / n_cg;         // k-steps of S per warp of a row group
        const int kk_lo = chunk * ks_per * 16, kk_hi = min(row, kk_lo + ks_per * 16);
#pragma unroll 2
        for (int kk = kk_lo; kk < kk_hi; kk += 16) {
            uint32_t a[4], b[LM_KT / 16][4];
            lm_ldmatrix_x4(a, q_s + (warp * 16 + (lane & 15)) * ld + kk + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < LM_KT / 16; ++j)
                lm_ldmatrix_x4(b[j], kt + (j * 16 + (lane & 7) + ((lane >> 4) << 3)) * ld + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int i = 0; i < LM_KT / 8; ++i) lm_mma(s[i], a, b[i >> 1][(i & 1) * 2], b[i >> 1][(i & 1) * 2 + 1]);
        }
        if (n_cg > 1) {
            // every warp of the row group gets the whole sums: its own part and the others', in the groups' order
            float* mine = sx + (size_t)((warp * n_cg + chunk) * 16) * 32;
#pragma unroll
            for (int i = 0; i < LM_KT / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) mine[(i * 4 + e) * 32 + lane] = s[i][e];
            asm volatile("bar.sync %0, %1;" ::"r"(1 + warp), "r"(32 * n_cg) : "memory");
#pragma unroll
            for (int i = 0; i < LM_KT / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
            for (int c = 0; c < n_cg; ++c) {
                const float* part = sx + (size_t)((warp * n_cg + c) * 16) * 32 + lane;
#pragma unroll
                for (int i = 0; i < LM_KT / 8; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[i][e] += part[(i * 4 + e) * 32];
            }
        }
        // mask, and the tile's row maxima
        const int pos0 = k_al + tile * LM_KT;
        float mx[2] = {-INFINITY, -INFINITY};
        // a tile that every token of the CTA sees whole (after the last token's window starts, before the first token's
        // own position ends) needs no mask
        const bool whole = pos0 + LM_KT - 1 <= p_first && (window <= 0 || pos0 >= k_hi - window + 1);
#pragma unroll
        for (int i = 0; i < LM_KT / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int u = e >> 1;
                bool ok = live[u];
                if (!whole) {
                    const int pos = pos0 + i * 8 + (lane & 3) * 2 + (e & 1);
                    ok = ok && pos >= lo_row[u] && pos <= p_row[u];
                }
                s[i][e] = ok ? s[i][e] * scale_log2 : -INFINITY;
                mx[u] = fmaxf(mx[u], s[i][e]);
            }
        float alpha[2], base[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            mx[u] = fmaxf(mx[u], __shfl_xor_sync(0xffffffffu, mx[u], 1));
            mx[u] = fmaxf(mx[u], __shfl_xor_sync(0xffffffffu, mx[u], 2));
            const float m_new = fmaxf(m[u], mx[u]);
            base[u] = m_new == -INFINITY ? 0.f : m_new;          // a row without a key so far: every term is zero
            alpha[u] = exp2f(m[u] - base[u]);
            m[u] = m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < LM_KT / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = exp2f(s[i][e] - base[e >> 1]);
                s[i][e] = p;
                sum[e >> 1] += p;
            }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], 1);
            sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], 2);
            l[u] = l[u] * alpha[u] + sum[u];
        }
        // the maxima seldom move after the first tiles: rescale only when a row of the warp needs it
        if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
            for (int i = 0; i < LM_DV / 8; ++i) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
        }
        // O += P V: the tile's rows again, their entries c0 .. as values
#pragma unroll
        for (int kk = 0; kk < LM_KT / 16; ++kk) {
            uint32_t a[4];
            a[0] = lm_pack(s[2 * kk][0], s[2 * kk][1]);
            a[1] = lm_pack(s[2 * kk][2], s[2 * kk][3]);
            a[2] = lm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = lm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int i = 0; i < LM_DV / 8; i += 2) {
                if (i < nt_live) {
                    uint32_t b[4];
                    lm_ldmatrix_x4_trans(b, kt + (kk * 16 + (lane & 15)) * ld + c0 + i * 8 + (lane >> 4) * 8);
                    lm_mma(o[i], a, b[0], b[1]);
                    lm_mma(o[i + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();      // the buffer is loaded again two tiles on
    }

#pragma unroll
    for (int u = 0; u < 2; ++u) {
        if (!live[u]) continue;
        const int r = warp * 16 + (lane >> 2) + u * 8;
        const int tt = r / hg, hh = r - tt * hg;
        const size_t th = (size_t)(tok0 + tt) * nh + h0 + hh;
        if (n_splits == 1) {
            const float inv = 1.0f / l[u];
#pragma unroll
            for (int i = 0; i < LM_DV / 8; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = c0 + i * 8 + (lane & 3) * 2 + e;
                    if (c < rank) out[th * rank + c] = __float2bfloat16_rn(o[i][u * 2 + e] * inv);
                }
        } else {
            float* po = part_o + (th * n_splits + split) * rank;
#pragma unroll
            for (int i = 0; i < LM_DV / 8; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = c0 + i * 8 + (lane & 3) * 2 + e;
                    if (c < rank) po[c] = o[i][u * 2 + e];
                }
            if (chunk == 0 && (lane & 3) == 0) {
                part_ml[(th * n_splits + split) * 2] = m[u];
                part_ml[(th * n_splits + split) * 2 + 1] = l[u];
            }
        }
    }
}

// out[t, h] = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m): the shares of one (token, head); maxima are base-2 exponents
__global__ void latent_combine_kernel(const float* part_o, const float* part_ml, __nv_bfloat16* out, int n_splits, int rank) {
    pdl_trigger();
    pdl_wait();
    const size_t th = blockIdx.x;
    const float* ml = part_ml + th * n_splits * 2;
    float mx = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, ml[2 * s]);
    float denom = 0.f;
    for (int s = 0; s < n_splits; ++s) denom += ml[2 * s] == -INFINITY ? 0.f : ml[2 * s + 1] * exp2f(ml[2 * s] - mx);
    const float inv = 1.0f / denom;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s)
            if (ml[2 * s] != -INFINITY) acc = fmaf(part_o[(th * n_splits + s) * rank + c], exp2f(ml[2 * s] - mx), acc);
        out[th * rank + c] = __float2bfloat16_rn(acc * inv);
    }
}

// n_tiles: an upper bound of the row tiles over the entries this launch takes (sum of ceil(len / (64 / hg)));
// max_len > 0: only entries of at most that many tokens.  part_o [T, nh, n_splits, rank], part_ml [T, nh, n_splits, 2].
PYRE_API int pyre_latent_attention_mma(const void* qa, const void* cache, void* out, float* part_o, float* part_ml,
                                       const int* block_table, int bt_stride, const int* cu_seqlens, const int* positions,
                                       int n_tokens, int n_seqs, int n_tiles, int nh, int rank, int row, int page_size, int window,
                                       float scale, int n_splits, int max_len, long long n_pages, int* err_flag,
                                       cudaStream_t stream) {
    if (n_tokens <= 0 || n_tiles <= 0) return 0;
    if (rank <= 0 || row < rank || row % 16 || nh <= 0 || page_size <= 0 || n_splits < 1) return PYRE_ERR_BAD_ARG;
    if (n_splits > 1 && (!part_o || !part_ml)) return PYRE_ERR_BAD_ARG;
    const int hg = min(nh, LM_ROWS);
    const int chunks = ceil_div(rank, LM_DV);
    if (chunks > 4) return PYRE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(LM_ROWS + 2 * LM_KT) * (row + 8) * sizeof(__nv_bfloat16) + (chunks > 1 ? (size_t)4 * chunks * 16 * 32 * sizeof(float) : 0);
    if (smem > 200 * 1024) return PYRE_ERR_UNSUPPORTED;
    static bool attr_set[PYRE_MAX_DEVICES] = {};
    const int dev = pyre_current_device();
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    const float scale_log2 = scale * 1.4426950408889634f;
    pyre_launch(latent_attention_mma_kernel, dim3(n_tiles, ceil_div(nh, hg), n_splits), dim3(128 * chunks), smem, stream,
                (const __nv_bfloat16*)qa, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, part_o, part_ml, block_table, bt_stride,
                cu_seqlens, positions, n_seqs, nh, hg, rank, row, page_size, window, scale_log2, n_splits, max_len, n_pages,
                err_flag);
    PYRE_LAUNCH_CHECK();
    if (n_splits > 1) {
        pyre_launch(latent_combine_kernel, dim3(n_tokens * nh), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml,
                    (__nv_bfloat16*)out, n_splits, rank);
        PYRE_LAUNCH_CHECK();
    }
    return 0;
}
