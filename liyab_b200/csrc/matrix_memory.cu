// Mixers whose memory is a matrix per head, carried from token to token:
//     S_t = keep_t S_{t-1} + take_t k_t v_t^T,      o_t = S_t^T q_t (over a normaliser, where the mixer has one).
// Two kinds of (keep, take):
//   fixed decay    keep = decay[h], take = 1, no normaliser (retention);
//   gated          from two numbers a token and head, i (log of the input gate) and f (log of the forget gate), with a
//                  running maximum m that starts at 0: m_t = max(f_t + m_{t-1}, i_t), keep = exp(f_t + m_{t-1} - m_t),
//                  take = exp(i_t - m_t); a vector n_t follows the same recurrence with k alone, and
//                  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).  The gates arrive as pre-activations:
//                  i = cap tanh(zi / cap), f = logsigmoid(cap tanh(zf / cap)).
// Queries and keys may be rotated first (the first rot_dims values of a head in pairs (j, j + rot_dims/2), angle =
// position * freq[j]) and scaled.  State, gates, angles and every sum are 32-bit.
//
// State of a request: [head][value tile][D x VT | D | 1] floats (S for the tile's VT value columns, n, m); every tile
// keeps its own n and m, so that the blocks of a launch share nothing.
//
// lb_matrix_memory walks a request's rows one after the other (a block per (request, head, value tile)); a decode step
// is one such row.  lb_matrix_memory_chunks does the same in pieces of 32 rows: inside a piece the rows' sums are
// products of small matrices (scores q_t . k_j weighted by the decay between j and t, then the values), and the state
// moves once per piece.
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

struct MemoryArgs {
    const float* q;            // [T, ld] rows, head h at columns h * D
    const float* k;
    const float* v;            // head h at columns h * E
    const float* zi;           // [T, ld] gate pre-activations, head h at column h (gated kind), else null
    const float* zf;
    int64_t ld;
    const float* decay;        // [H] (fixed kind), else null
    const float* freq;         // [rot_dims / 2] or null
    const int32_t* positions;  // [T]
    const int32_t* q_start;    // [S + 1]
    const int32_t* slots;      // [S]
    float* state;              // [slot][H][NV][D * VT + D + 1]
    int64_t slot_stride;       // floats per slot
    float* out;                // [T, ldo], head h at columns h * E
    int64_t ldo;
    int H, D, E, VT, NV, rot_dims;
    float q_scale, k_scale, cap;
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

// Value d of a head's query or key row for the token at `pos`, rotated and scaled.
__device__ __forceinline__ float rotated(const float* row, int d, int rot_dims, const float* freq, int pos, float scale) {
    float v = row[d];
    if (d < rot_dims) {
        const int half = rot_dims >> 1, j = d < half ? d : d - half;
        float sn, cs;
        sincosf((float)pos * freq[j], &sn, &cs);
        const float lo = row[j], hi = row[j + half];
        v = d < half ? lo * cs - hi * sn : hi * cs + lo * sn;
    }
    return v * scale;
}

// The two gates of a token and head and the maximum after them.
__device__ __forceinline__ void gates(const MemoryArgs& a, int row, int h, float m_prev, float* keep, float* take, float* m_new) {
    if (a.decay != nullptr) {
        *keep = a.decay[h];
        *take = 1.0f;
        *m_new = 0.0f;
        return;
    }
    const float gi = a.cap * tanhf(a.zi[(size_t)row * a.ld + h] / a.cap);
    const float gf = log_sigmoid(a.cap * tanhf(a.zf[(size_t)row * a.ld + h] / a.cap));
    const float m = fmaxf(gf + m_prev, gi);
    *keep = expf(gf + m_prev - m);
    *take = expf(gi - m);
    *m_new = m;
}

// ---------------------------------------------------------------- row by row
// 256 threads: thread (c, ds) owns rows ds, ds + DS, .. of column c of the tile's S (in shared memory).
__global__ void __launch_bounds__(256) matrix_memory_rows_kernel(MemoryArgs a, int vt_pow2) {
    extern __shared__ float smem[];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int seq = blockIdx.x, h = blockIdx.y, nv = blockIdx.z;
    const int row0 = a.q_start[seq], row1 = a.q_start[seq + 1];
    if (row1 <= row0) return;
    const int D = a.D, VT = a.VT, E = a.E;
    const int c = threadIdx.x & (vt_pow2 - 1), ds = threadIdx.x / vt_pow2, DS = blockDim.x / vt_pow2;
    const int col = nv * VT + c;
    const bool live = c < VT && col < E;
    float* S = smem;                       // [D][VT]
    float* ns = S + (size_t)D * VT;        // [D]
    float* qs = ns + D;                    // [D]
    float* ks = qs + D;                    // [D]
    float* red = ks + D;                   // [DS][vt_pow2]
    float* st = a.state + (size_t)a.slots[seq] * a.slot_stride + ((size_t)h * a.NV + nv) * ((size_t)D * VT + D + 1);
    const bool gated = a.decay == nullptr;
    for (int i = threadIdx.x; i < D * VT + D; i += blockDim.x) S[i] = st[i];       // S and n lie one after the other
    float m = st[(size_t)D * VT + D];
    __syncthreads();
    for (int row = row0; row < row1; ++row) {
        const int pos = a.positions[row];
        float keep, take, m_new;
        gates(a, row, h, m, &keep, &take, &m_new);
        m = m_new;
        for (int d = threadIdx.x; d < 2 * D; d += blockDim.x) {
            const bool is_k = d >= D;
            const int dd = is_k ? d - D : d;
            const float* src = (is_k ? a.k : a.q) + (size_t)row * a.ld + (size_t)h * D;
            (is_k ? ks : qs)[dd] = rotated(src, dd, a.rot_dims, a.freq, pos, is_k ? a.k_scale : a.q_scale);
        }
        __syncthreads();
        float acc = 0.0f;
        if (live) {
            const float tv = take * a.v[(size_t)row * a.ld + (size_t)h * E + col];
            for (int d = ds; d < D; d += DS) {
                const float s = fmaf(keep, S[d * VT + c], ks[d] * tv);
                S[d * VT + c] = s;
                acc = fmaf(s, qs[d], acc);
            }
        }
        red[ds * vt_pow2 + c] = acc;
        if (gated)
            for (int d = threadIdx.x; d < D; d += blockDim.x) ns[d] = fmaf(keep, ns[d], take * ks[d]);
        __syncthreads();
        if (ds == 0 && live) {
            float o = 0.0f;
            for (int i = 0; i < DS; ++i) o += red[i * vt_pow2 + c];
            if (gated) {
                float nq = 0.0f;
                for (int d = 0; d < D; ++d) nq = fmaf(ns[d], qs[d], nq);
                o /= fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
            }
            a.out[(size_t)row * a.ldo + (size_t)h * E + col] = o;
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < D * VT + D; i += blockDim.x) st[i] = S[i];
    if (threadIdx.x == 0) st[(size_t)D * VT + D] = m;
}

}  // namespace

extern "C" int lb_matrix_memory(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                                int64_t slot_stride, float* out, int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile, float q_scale,
                                float k_scale, float cap, int chunked, void* stream) {
    LB_CHECK_ARG(n_seq >= 0 && n_head > 0 && dim > 0 && vdim > 0 && value_tile > 0 && value_tile <= 64, "matrix memory: bad sizes heads=%d dim=%d vdim=%d tile=%d",
                 n_head, dim, vdim, value_tile);
    LB_CHECK_ARG((decay != nullptr) != (zi != nullptr && zf != nullptr), "matrix memory: either a fixed decay or the two gates");
    LB_CHECK_ARG(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || freq != nullptr), "matrix memory: %d of %d values to rotate", rot_dims, dim);
    if (n_seq == 0) return LB_OK;
    MemoryArgs a{};
    a.q = q; a.k = k; a.v = v; a.zi = zi; a.zf = zf; a.ld = ld; a.decay = decay; a.freq = freq; a.positions = positions; a.q_start = q_start;
    a.slots = slots; a.state = state; a.slot_stride = slot_stride; a.out = out; a.ldo = ldo;
    a.H = n_head; a.D = dim; a.E = vdim; a.VT = value_tile; a.NV = (vdim + value_tile - 1) / value_tile; a.rot_dims = rot_dims;
    a.q_scale = q_scale; a.k_scale = k_scale; a.cap = cap;
    LB_CHECK_ARG(slot_stride >= (int64_t)n_head * a.NV * ((int64_t)dim * value_tile + dim + 1), "matrix memory: the state slots are too small");
    int p2 = 1;
    while (p2 < value_tile) p2 <<= 1;
    auto s = static_cast<cudaStream_t>(stream);
    (void)chunked;
    const size_t smem = ((size_t)dim * value_tile + 3 * (size_t)dim + 256) * sizeof(float);
    LB_CHECK_ARG(smem <= 200 * 1024, "matrix memory: a tile of %d x %d floats does not fit shared memory", dim, value_tile);
    if (smem > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(matrix_memory_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LB_CHECK_CUDA(lb_launch_overlapped(matrix_memory_rows_kernel, dim3(n_seq, n_head, a.NV), dim3(256), smem, s, a, p2));
    return LB_OK;
}
