// Linear attention with a constant decay per head, as a recurrence over a state that lives in a slot of the
// cache manager:
//   S_t = decay_h S_(t-1) + k_t v_t^T        S: [dk, dv] fp32 per (request, head), zero when a request begins
//   o_t = S_t^T q_t                           no other scale
// with q, k (dk per head) and v (dv per head) taken from the token's projection row through an activation
// (0: none, 1: silu), computed in fp32 and rounded to the activations' type.  The state, the decay and every sum are fp32.
//
// This kernel walks the tokens of an entry one after the other: a prompt portion and a single decoded token
// are the same case, and the result is bit-identical however a request's tokens were cut into steps (the
// order of every sum is fixed by dk and the thread layout alone).
//
// Grid (tiles of 32 value columns, heads, entries); a CTA of four warps owns a [dk, 32] tile of the state in
// registers.  A warp holds eight columns; its lanes split the dk rows four ways in groups of four
// (row = 16 g + 4 r + e), so q and k come from shared memory as conflict-free 16-byte loads, and the four
// row groups of a column meet in two shuffles.  Tokens are staged through shared memory sixteen at a time.
#include "common.cuh"

namespace {

constexpr int LA_WARPS = 4;
constexpr int LA_COLS = 32;    // value columns per CTA
constexpr int LA_CHUNK = 16;   // tokens staged at a time

__device__ __forceinline__ float la_act(float z, int act) { return act == 1 ? z / (1.0f + expf(-z)) : z; }
// the activation's result in the activations' own type (bfloat16 rounds here, as the tensor-core kernel's operands do)
template <typename T> __device__ __forceinline__ float la_in(T x, int act) { return to_f32<T>(from_f32<T>(la_act(to_f32<T>(x), act))); }

// G: groups of 16 rows (dk <= 16 G); a thread holds 4 G state elements of one column
template <typename T, int G>
__global__ void __launch_bounds__(LA_WARPS * 32)
linear_attention_scan_kernel(const T* proj, long long row_stride, int q_col, int k_col, int v_col, float* state,
                             const int* slots, const int* cu_seqlens, const float* decay, float* out, int H, int dk,
                             int dv, int act, int max_len) {
    constexpr int DKP = 16 * G;
    __shared__ __align__(16) float sq[LA_CHUNK][DKP];
    __shared__ __align__(16) float sk[LA_CHUNK][DKP];
    __shared__ float sv[LA_CHUNK][LA_COLS];
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int jj = lane & 7, r = lane >> 3;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int col0 = blockIdx.x * LA_COLS;
    const int col = col0 + warp * 8 + jj;
    const bool col_ok = col < dv;
    const int tok0 = cu_seqlens[seq], tok1 = cu_seqlens[seq + 1];
    if (max_len > 0 && tok1 - tok0 > max_len) return;      // the whole CTA: such entries belong to the tensor-core kernel
    const float lam = decay[h];
    float* S_g = state + ((size_t)slots[seq] * H + h) * dk * dv;

    float S[4 * G];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 16 * g + 4 * r + e;
            S[4 * g + e] = (col_ok && i < dk) ? S_g[(size_t)i * dv + col] : 0.f;
        }

    for (int c0 = tok0; c0 < tok1; c0 += LA_CHUNK) {
        const int n = min(LA_CHUNK, tok1 - c0);
        __syncthreads();      // the last chunk's rows have been read
        for (int e = threadIdx.x; e < n * DKP; e += LA_WARPS * 32) {
            const int tt = e / DKP, i = e - tt * DKP;
            const T* row = proj + (size_t)(c0 + tt) * row_stride;
            sq[tt][i] = i < dk ? la_in<T>(row[q_col + (size_t)h * dk + i], act) : 0.f;
            sk[tt][i] = i < dk ? la_in<T>(row[k_col + (size_t)h * dk + i], act) : 0.f;
        }
        for (int e = threadIdx.x; e < n * LA_COLS; e += LA_WARPS * 32) {
            const int tt = e / LA_COLS, j = e - tt * LA_COLS;
            const T* row = proj + (size_t)(c0 + tt) * row_stride;
            sv[tt][j] = col0 + j < dv ? la_in<T>(row[v_col + (size_t)h * dv + col0 + j], act) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float vj = sv[tt][warp * 8 + jj];
            float acc = 0.f;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][16 * g + 4 * r]);
                const float4 q4 = *reinterpret_cast<const float4*>(&sq[tt][16 * g + 4 * r]);
                S[4 * g + 0] = fmaf(lam, S[4 * g + 0], k4.x * vj); acc = fmaf(S[4 * g + 0], q4.x, acc);
                S[4 * g + 1] = fmaf(lam, S[4 * g + 1], k4.y * vj); acc = fmaf(S[4 * g + 1], q4.y, acc);
                S[4 * g + 2] = fmaf(lam, S[4 * g + 2], k4.z * vj); acc = fmaf(S[4 * g + 2], q4.z, acc);
                S[4 * g + 3] = fmaf(lam, S[4 * g + 3], k4.w * vj); acc = fmaf(S[4 * g + 3], q4.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (r == 0 && col_ok) out[(size_t)(c0 + tt) * H * dv + (size_t)h * dv + col] = acc;
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 16 * g + 4 * r + e;
            if (col_ok && i < dk) S_g[(size_t)i * dv + col] = S[4 * g + e];
        }
}

}  // namespace

// proj: [n_tokens, row_stride] activations; state: one layer of a state buffer [slots][H][dk][dv] fp32;
// slots[b]: the slot of entry b; cu_seqlens [n_seqs + 1]; decay [H] fp32; out [n_tokens, H * dv] fp32.
// max_len > 0: only entries of at most that many tokens (longer ones go to pyre_linear_attention_chunked).
PYRE_API int pyre_linear_attention_scan(const void* proj, long long row_stride, int q_col, int k_col, int v_col,
                                        float* state, const int* slots, const int* cu_seqlens, const float* decay,
                                        float* out, int n_tokens, int n_seqs, int H, int dk, int dv, int act, int dtype,
                                        int max_len, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || dk > 256 || H > 65535 || n_seqs > 65535 || (act != 0 && act != 1)) return PYRE_ERR_UNSUPPORTED;
    const dim3 grid(ceil_div(dv, LA_COLS), H, n_seqs), block(LA_WARPS * 32);
#define LA_LAUNCH(TT, GG) pyre_launch(linear_attention_scan_kernel<TT, GG>, grid, block, 0, stream, (const TT*)proj, row_stride, q_col, k_col, v_col, state, slots, cu_seqlens, decay, out, H, dk, dv, act, max_len)
#define LA_PICK(TT) do { if (dk <= 16) LA_LAUNCH(TT, 1); else if (dk <= 32) LA_LAUNCH(TT, 2); else if (dk <= 64) LA_LAUNCH(TT, 4); \
                         else if (dk <= 128) LA_LAUNCH(TT, 8); else LA_LAUNCH(TT, 16); } while (0)
    if (dtype == PYRE_BF16) LA_PICK(__nv_bfloat16);
    else if (dtype == PYRE_F32) LA_PICK(float);
    else return PYRE_ERR_BAD_ARG;
#undef LA_PICK
#undef LA_LAUNCH
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// The same recurrence for prompt portions, on the tensor cores, in chunks of 64 tokens (query/key size 64) or 128
// tokens (query/key size 128) (bfloat16 activations).
// For the tokens i, j of a chunk that starts from the state S (n tokens, w = decay):
//   A[i][j] = (q_i . k_j) w^(i-j)  for j <= i, else 0                       (fp32 scores, decays applied in fp32)
//   o_i     = sum_j A[i][j] v_j  +  w^(i+1) S^T q_i
//   S'      = w^n S + sum_j k_j (w^(n-1-j) v_j)^T
// Every product is an mma.sync m16n8k16 of bf16 operands with fp32 accumulators.  Operands that exist only in
// fp32 (the masked scores A, the state S, the decayed values) enter as a sum of two bf16 numbers (value rounded,
// and the remainder rounded: 16 bits of mantissa), so they are not rounded to 8 bits on the way.  q, k and v
// are silu(projection) rounded to bf16 once.
//
// Grid (tiles of 32 value columns, heads, entries); four or eight warps.  Warp w owns the chunk's tokens 16 w .. 16 w + 15
// for the outputs, and 16 rows of the state tile [DK, 32], which it keeps in MMA accumulator
// registers; the state's two bf16 halves are left in shared memory for the other warps' q S products.  The next
// chunk's q, k, v rows arrive by cp.async while a chunk is computed.  Entries shorter than min_len are left to
// the scan kernel.  The result differs from the scan's by rounding only.
// ---------------------------------------------------------------------------
namespace {

constexpr int LC_COLS = 32;
constexpr int LC_VP = LC_COLS + 8;      // pitch of the value and state tiles in shared memory (elements)

__device__ __forceinline__ void lc_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lc_ldsm(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lc_ldsm_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t lc_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// x = hi + lo with hi = bf16(x), lo = bf16(x - hi), for a pair of values
__device__ __forceinline__ void lc_split(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
    hi = lc_pack(__bfloat162float(h0), __bfloat162float(h1));
    lo = lc_pack(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
}
__device__ __forceinline__ void lc_cp16(uint32_t dst, const void* src, bool real) {
    const int n = real ? 16 : 0;      // 0 bytes read: the 16 bytes at dst become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

// silu for operands that are rounded to bfloat16 at once: the fast exponential and division are exact enough
__device__ __forceinline__ float lc_silu(float z) { return __fdividef(z, 1.0f + __expf(-z)); }

// WARPS warps; a chunk is 16 WARPS tokens (64 or 128)
template <int DK, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
linear_attention_chunk_kernel(const __nv_bfloat16* proj, long long row_stride, int q_col, int k_col, int v_col, float* state,
                              const int* slots, const int* cu_seqlens, const float* decay, float* out, int H, int dv,
                              int act, int min_len) {
    constexpr int QP = DK + 8;            // pitch of the q and k tiles (elements): rows 16 bytes apart in banks
    constexpr int LC_CHUNK = 16 * WARPS, NTH = 32 * WARPS;
    constexpr int MT = DK / LC_CHUNK;     // 16-row tiles of the state per warp
    static_assert(MT >= 1 && MT * LC_CHUNK == DK, "every warp owns whole 16-row tiles of the state");
    extern __shared__ __align__(16) unsigned char lc_smem[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(lc_smem);                 // [2][64][QP]
    __nv_bfloat16* sK = sQ + 2 * LC_CHUNK * QP;                                    // [2][64][QP]
    __nv_bfloat16* sV = sK + 2 * LC_CHUNK * QP;                                    // [2][64][LC_VP]
    __nv_bfloat16* sSh = sV + 2 * LC_CHUNK * LC_VP;                                // [DK][LC_VP] state, rounded
    __nv_bfloat16* sSl = sSh + DK * LC_VP;                                         // [DK][LC_VP] state, remainder
    float* pw = reinterpret_cast<float*>(sSl + DK * LC_VP);                        // [chunk + 1] powers of the decay
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.y, seq = blockIdx.z, col0 = blockIdx.x * LC_COLS;
    const int tok0 = cu_seqlens[seq], tok1 = cu_seqlens[seq + 1];
    if (tok1 - tok0 < min_len) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const float lam = decay[h];
    float* S_g = state + ((size_t)slots[seq] * H + h) * DK * dv + col0;
    const __nv_bfloat16* q_src = proj + q_col + (size_t)h * DK;
    const __nv_bfloat16* k_src = proj + k_col + (size_t)h * DK;
    const __nv_bfloat16* v_src = proj + v_col + (size_t)h * dv + col0;

    auto load_chunk = [&](int stage, int c0) {
        const int n = min(LC_CHUNK, tok1 - c0);
        __nv_bfloat16* q = sQ + stage * LC_CHUNK * QP;
        __nv_bfloat16* k = sK + stage * LC_CHUNK * QP;
        __nv_bfloat16* v = sV + stage * LC_CHUNK * LC_VP;
        for (int e = threadIdx.x; e < LC_CHUNK * (DK / 8); e += NTH) {
            const int r = e / (DK / 8), c = (e - r * (DK / 8)) * 8;
            const size_t row = (size_t)(c0 + (r < n ? r : 0)) * row_stride;
            lc_cp16((uint32_t)__cvta_generic_to_shared(q + r * QP + c), q_src + row + c, r < n);
            lc_cp16((uint32_t)__cvta_generic_to_shared(k + r * QP + c), k_src + row + c, r < n);
        }
        for (int e = threadIdx.x; e < LC_CHUNK * (LC_COLS / 8); e += NTH) {
            const int r = e / (LC_COLS / 8), c = (e - r * (LC_COLS / 8)) * 8;
            const size_t row = (size_t)(c0 + (r < n ? r : 0)) * row_stride;
            lc_cp16((uint32_t)__cvta_generic_to_shared(v + r * LC_VP + c), v_src + row + c, r < n);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    load_chunk(0, tok0);

    if (threadIdx.x == 0) {
        float p = 1.f;
        for (int i = 0; i <= LC_CHUNK; ++i) { pw[i] = p; p *= lam; }
    }
    // this warp's rows of the state tile, as accumulator fragments: element (row m0 + 16 mt + g (+ 8), column 8 nt + 2 t (+ 1))
    const int m0 = warp * (DK / WARPS);
    float S[MT][4][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float* p0 = S_g + (size_t)(m0 + 16 * mt + g) * dv + 8 * nt + 2 * t;
            const float2 lo = *reinterpret_cast<const float2*>(p0), hi = *reinterpret_cast<const float2*>(p0 + (size_t)8 * dv);
            S[mt][nt][0] = lo.x; S[mt][nt][1] = lo.y; S[mt][nt][2] = hi.x; S[mt][nt][3] = hi.y;
        }
    auto publish_state = [&]() {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                uint32_t h0, l0, h1, l1;
                lc_split(S[mt][nt][0], S[mt][nt][1], h0, l0);
                lc_split(S[mt][nt][2], S[mt][nt][3], h1, l1);
                const int at = (m0 + 16 * mt + g) * LC_VP + 8 * nt + 2 * t;
                *reinterpret_cast<uint32_t*>(sSh + at) = h0; *reinterpret_cast<uint32_t*>(sSl + at) = l0;
                *reinterpret_cast<uint32_t*>(sSh + at + 8 * LC_VP) = h1; *reinterpret_cast<uint32_t*>(sSl + at + 8 * LC_VP) = l1;
            }
    };
    publish_state();

    int stage = 0;
    for (int c0 = tok0; c0 < tok1; c0 += LC_CHUNK, stage ^= 1) {
        const int n = min(LC_CHUNK, tok1 - c0);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();      // this chunk's rows are here; the state's halves and the powers are published
        if (c0 + LC_CHUNK < tok1) load_chunk(stage ^ 1, c0 + LC_CHUNK);
        __nv_bfloat16* q = sQ + stage * LC_CHUNK * QP;
        __nv_bfloat16* k = sK + stage * LC_CHUNK * QP;
        __nv_bfloat16* v = sV + stage * LC_CHUNK * LC_VP;
        if (act == 1) {
            for (int e = threadIdx.x; e < LC_CHUNK * (DK / 2); e += NTH) {
                const int r = e / (DK / 2), c = (e - r * (DK / 2)) * 2;
                __nv_bfloat162* pq = reinterpret_cast<__nv_bfloat162*>(q + r * QP + c);
                __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(k + r * QP + c);
                const float2 a = __bfloat1622float2(*pq), b = __bfloat1622float2(*pk);
                *pq = __floats2bfloat162_rn(lc_silu(a.x), lc_silu(a.y));
                *pk = __floats2bfloat162_rn(lc_silu(b.x), lc_silu(b.y));
            }
            for (int e = threadIdx.x; e < LC_CHUNK * (LC_COLS / 2); e += NTH) {
                const int r = e / (LC_COLS / 2), c = (e - r * (LC_COLS / 2)) * 2;
                __nv_bfloat162* pv = reinterpret_cast<__nv_bfloat162*>(v + r * LC_VP + c);
                const float2 a = __bfloat1622float2(*pv);
                *pv = __floats2bfloat162_rn(lc_silu(a.x), lc_silu(a.y));
            }
            __syncthreads();
        }
        const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(q), k_s = (uint32_t)__cvta_generic_to_shared(k);
        const uint32_t v_s = (uint32_t)__cvta_generic_to_shared(v);
        const uint32_t sh_s = (uint32_t)__cvta_generic_to_shared(sSh), sl_s = (uint32_t)__cvta_generic_to_shared(sSl);
        const int i0 = 16 * warp;      // this warp's tokens of the chunk

        // ---- scores of this warp's 16 tokens against the chunk's keys up to its own (later keys are masked anyway),
        // and q S for the same tokens; a warp whose tokens lie beyond the portion's end has nothing to do here
        if (i0 < n) {
        float sc[2 * WARPS][4], oi[4][4];
#pragma unroll
        for (int nt = 0; nt < 2 * WARPS; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) { oi[nt][0] = oi[nt][1] = oi[nt][2] = oi[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            uint32_t a[4];
            lc_ldsm(a, q_s + (uint32_t)(((i0 + (lane & 7) + ((lane >> 3) & 1) * 8) * QP + 16 * ks + (lane >> 4) * 8) * 2));
#pragma unroll
            for (int np = 0; np < WARPS; ++np) {       // keys 16 np .. 16 np + 15
                if (np > warp) continue;
                uint32_t b[4];
                lc_ldsm(b, k_s + (uint32_t)(((16 * np + (lane & 7) + (lane >> 4) * 8) * QP + 16 * ks + ((lane >> 3) & 1) * 8) * 2));
                lc_mma(sc[2 * np], a, b[0], b[1]);
                lc_mma(sc[2 * np + 1], a, b[2], b[3]);
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {       // state rows 16 ks .., columns 16 np .. 16 np + 15, both halves
                uint32_t bh[4], bl[4];
                const uint32_t off = (uint32_t)(((16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8) * LC_VP + 16 * np + (lane >> 4) * 8) * 2);
                lc_ldsm_t(bh, sh_s + off);
                lc_ldsm_t(bl, sl_s + off);
                lc_mma(oi[2 * np], a, bh[0], bh[1]); lc_mma(oi[2 * np], a, bl[0], bl[1]);
                lc_mma(oi[2 * np + 1], a, bh[2], bh[3]); lc_mma(oi[2 * np + 1], a, bl[2], bl[3]);
            }
        }
        // ---- the decays of the chunk: A[i][j] = score w^(i - j) for j <= i; the rows of q S get w^(i + 1)
        const int ia = i0 + g, ib = ia + 8;
        float o[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float wa = pw[ia + 1], wb = pw[ib + 1];
            o[nt][0] = oi[nt][0] * wa; o[nt][1] = oi[nt][1] * wa; o[nt][2] = oi[nt][2] * wb; o[nt][3] = oi[nt][3] * wb;
        }
#pragma unroll
        for (int nt = 0; nt < 2 * WARPS; ++nt) {
            const int j = 8 * nt + 2 * t;
            sc[nt][0] = j <= ia ? sc[nt][0] * pw[ia - j] : 0.f;
            sc[nt][1] = j + 1 <= ia ? sc[nt][1] * pw[ia - j - 1] : 0.f;
            sc[nt][2] = j <= ib ? sc[nt][2] * pw[ib - j] : 0.f;
            sc[nt][3] = j + 1 <= ib ? sc[nt][3] * pw[ib - j - 1] : 0.f;
        }
        // ---- o += A v  (A as two bf16 halves; keys 16 kk .. 16 kk + 15 per step)
#pragma unroll
        for (int kk = 0; kk < WARPS; ++kk) {
            if (kk > warp) continue;
            uint32_t ah[4], al[4];
            lc_split(sc[2 * kk][0], sc[2 * kk][1], ah[0], al[0]);
            lc_split(sc[2 * kk][2], sc[2 * kk][3], ah[1], al[1]);
            lc_split(sc[2 * kk + 1][0], sc[2 * kk + 1][1], ah[2], al[2]);
            lc_split(sc[2 * kk + 1][2], sc[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b[4];
                lc_ldsm_t(b, v_s + (uint32_t)(((16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8) * LC_VP + 16 * np + (lane >> 4) * 8) * 2));
                lc_mma(o[2 * np], ah, b[0], b[1]); lc_mma(o[2 * np], al, b[0], b[1]);
                lc_mma(o[2 * np + 1], ah, b[2], b[3]); lc_mma(o[2 * np + 1], al, b[2], b[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float* dst = out + (size_t)(c0 + ia) * H * dv + (size_t)h * dv + col0 + 8 * nt + 2 * t;
            if (ia < n) *reinterpret_cast<float2*>(dst) = make_float2(o[nt][0], o[nt][1]);
            if (ib < n) *reinterpret_cast<float2*>(dst + (size_t)8 * H * dv) = make_float2(o[nt][2], o[nt][3]);
        }
        }
        __syncthreads();      // every warp has read the old state's halves
        // ---- the state after the chunk: S = w^n S + K^T (w^(n - 1 - j) v_j)
        const float wn = pw[n];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                S[mt][nt][0] *= wn; S[mt][nt][1] *= wn; S[mt][nt][2] *= wn; S[mt][nt][3] *= wn;
            }
#pragma unroll
        for (int kk = 0; kk < WARPS; ++kk) {
            if (16 * kk >= n) continue;
            // the decayed values of tokens 16 kk .., as B fragments in two halves: a lane holds tokens 16 kk + 2 t (+ 1) (+ 8)
            const int j0 = 16 * kk + 2 * t;
            const float w0 = j0 < n ? pw[n - 1 - j0] : 0.f, w1 = j0 + 1 < n ? pw[n - 2 - j0] : 0.f;
            const float w2 = j0 + 8 < n ? pw[n - 9 - j0] : 0.f, w3 = j0 + 9 < n ? pw[n - 10 - j0] : 0.f;
            uint32_t bh[4][2], bl[4][2];
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b[4];
                lc_ldsm_t(b, v_s + (uint32_t)(((16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8) * LC_VP + 16 * np + (lane >> 4) * 8) * 2));
#pragma unroll
                for (int u = 0; u < 2; ++u) {      // value columns 16 np + 8 u ..
                    const float2 x = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&b[2 * u]));
                    const float2 y = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&b[2 * u + 1]));
                    lc_split(x.x * w0, x.y * w1, bh[2 * np + u][0], bl[2 * np + u][0]);
                    lc_split(y.x * w2, y.y * w3, bh[2 * np + u][1], bl[2 * np + u][1]);
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                // K^T: rows are this warp's state rows (dims of k), the inner index is the token: the tile is read transposed
                uint32_t a[4];
                const int mi = lane >> 3;
                lc_ldsm_t(a, k_s + (uint32_t)(((16 * kk + (lane & 7) + (mi >> 1) * 8) * QP + m0 + 16 * mt + (mi & 1) * 8) * 2));
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    lc_mma(S[mt][nt], a, bh[nt][0], bh[nt][1]);
                    lc_mma(S[mt][nt], a, bl[nt][0], bl[nt][1]);
                }
            }
        }
        publish_state();
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float* p0 = S_g + (size_t)(m0 + 16 * mt + g) * dv + 8 * nt + 2 * t;
            *reinterpret_cast<float2*>(p0) = make_float2(S[mt][nt][0], S[mt][nt][1]);
            *reinterpret_cast<float2*>(p0 + (size_t)8 * dv) = make_float2(S[mt][nt][2], S[mt][nt][3]);
        }
}

template <int DK, int WARPS>
int lc_launch(dim3 grid, cudaStream_t stream, const __nv_bfloat16* proj, long long row_stride, int q_col, int k_col, int v_col,
              float* state, const int* slots, const int* cu_seqlens, const float* decay, float* out, int H, int dv, int act, int min_len) {
    constexpr int LC_CHUNK = 16 * WARPS;
    constexpr size_t SMEM = (size_t)(4 * LC_CHUNK * (DK + 8) + 2 * LC_CHUNK * LC_VP + 2 * DK * LC_VP) * 2 + (LC_CHUNK + 8) * sizeof(float);
    static bool configured_on[PYRE_MAX_DEVICES] = {};
    bool& configured = configured_on[pyre_current_device()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_attention_chunk_kernel<DK, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    pyre_launch(linear_attention_chunk_kernel<DK, WARPS>, grid, dim3(WARPS * 32), SMEM, stream, proj, row_stride, q_col, k_col, v_col, state, slots,
                cu_seqlens, decay, out, H, dv, act, min_len);
    return (int)cudaGetLastError();
}

}  // namespace

// Can pyre_linear_attention_chunked take these sizes?  Query/key sizes 64 and 128, value sizes that are multiples
// of 32, and rows, columns and heads that start on 16-byte boundaries (cp.async copies of eight elements).
static inline int linear_attention_chunked_ok(long long row_stride, int q_col, int k_col, int v_col, int dk, int dv) {
    return (dk == 64 || dk == 128) && dv % 32 == 0 && row_stride % 8 == 0 && q_col % 8 == 0 && k_col % 8 == 0 && v_col % 8 == 0;
}

// The entries of at least min_len tokens (bfloat16 activations); arguments as pyre_linear_attention_scan.
PYRE_API int pyre_linear_attention_chunked(const void* proj, long long row_stride, int q_col, int k_col, int v_col,
                                           float* state, const int* slots, const int* cu_seqlens, const float* decay,
                                           float* out, int n_tokens, int n_seqs, int H, int dk, int dv, int act, int min_len,
                                           cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (!linear_attention_chunked_ok(row_stride, q_col, k_col, v_col, dk, dv) || ((uintptr_t)proj & 15) || ((uintptr_t)state & 7) ||
        ((uintptr_t)out & 7) || H <= 0 || H > 65535 || n_seqs > 65535 || (act != 0 && act != 1) || min_len < 1)
        return PYRE_ERR_UNSUPPORTED;
    const dim3 grid(dv / LC_COLS, H, n_seqs);
    const __nv_bfloat16* p = (const __nv_bfloat16*)proj;
    return dk == 64 ? lc_launch<64, 4>(grid, stream, p, row_stride, q_col, k_col, v_col, state, slots, cu_seqlens, decay, out, H, dv, act, min_len)
                    : lc_launch<128, 8>(grid, stream, p, row_stride, q_col, k_col, v_col, state, slots, cu_seqlens, decay, out, H, dv, act, min_len);
}
