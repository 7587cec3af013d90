// Linear attention with a constant decay per head, as a recurrence over a state that lives in a slot of the
// cache manager:
//   S_t = decay_h S_(t-1) + k_t v_t^T        S: [dk, dv] fp32 per (request, head), zero when a request begins
//   o_t = S_t^T q_t                           no other scale
// with q, k (dk per head) and v (dv per head) taken from the token's projection row through an activation
// (0: none, 1: silu), computed in fp32.  The state, the decay and every sum are fp32.
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

// G: groups of 16 rows (dk <= 16 G); a thread holds 4 G state elements of one column
template <typename T, int G>
__global__ void __launch_bounds__(LA_WARPS * 32)
linear_attention_scan_kernel(const T* proj, long long row_stride, int q_col, int k_col, int v_col, float* state,
                             const int* slots, const int* cu_seqlens, const float* decay, float* out, int H, int dk,
                             int dv, int act) {
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
            sq[tt][i] = i < dk ? la_act(to_f32<T>(row[q_col + (size_t)h * dk + i]), act) : 0.f;
            sk[tt][i] = i < dk ? la_act(to_f32<T>(row[k_col + (size_t)h * dk + i]), act) : 0.f;
        }
        for (int e = threadIdx.x; e < n * LA_COLS; e += LA_WARPS * 32) {
            const int tt = e / LA_COLS, j = e - tt * LA_COLS;
            const T* row = proj + (size_t)(c0 + tt) * row_stride;
            sv[tt][j] = col0 + j < dv ? la_act(to_f32<T>(row[v_col + (size_t)h * dv + col0 + j]), act) : 0.f;
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
PYRE_API int pyre_linear_attention_scan(const void* proj, long long row_stride, int q_col, int k_col, int v_col,
                                        float* state, const int* slots, const int* cu_seqlens, const float* decay,
                                        float* out, int n_tokens, int n_seqs, int H, int dk, int dv, int act, int dtype,
                                        cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || dk > 256 || H > 65535 || n_seqs > 65535 || (act != 0 && act != 1)) return PYRE_ERR_UNSUPPORTED;
    const dim3 grid(ceil_div(dv, LA_COLS), H, n_seqs), block(LA_WARPS * 32);
#define LA_LAUNCH(TT, GG) pyre_launch(linear_attention_scan_kernel<TT, GG>, grid, block, 0, stream, (const TT*)proj, row_stride, q_col, k_col, v_col, state, slots, cu_seqlens, decay, out, H, dk, dv, act)
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
