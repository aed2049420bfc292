// Row-wise pieces that sit between the matrix products of a block: the RMS norm in groups, the blend of a
// token's normalised row with the row before it (token shift, with the last row of every request kept as state),
// the xIELU activation, and the gated per-token side input.  Statistics, blends and activations are 32-bit
// whatever the element type of the rows.
#include "api.h"
#include "common.cuh"

namespace {

// ---------------------------------------------------------------- RMS norm in groups
// The row is cut into `groups` equal consecutive parts; y = x / sqrt(mean(part^2) + eps) * w.  One block per
// (row, group); the sum's order depends on the part's length alone.  `gain_offset` is added to every gain (1 for gains
// that are stored around zero, else 0).
template <typename T>
__global__ void rms_groups_kernel(const float* __restrict__ x, int64_t ldx, const int32_t* __restrict__ rows, const float* __restrict__ w,
                                  T* __restrict__ y, int64_t ldy, int part, float eps, float gain_offset) {
    __shared__ float scratch[33];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int r = blockIdx.x, g = blockIdx.y;
    const float* in = x + (size_t)(rows != nullptr ? rows[r] : r) * ldx + (size_t)g * part;
    const float* gain = w != nullptr ? w + (size_t)g * part : nullptr;
    T* out = y + (size_t)r * ldy + (size_t)g * part;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    const float inv = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float v = in[i] * inv;
        if (gain != nullptr) v *= gain[i] + gain_offset;
        out[i] = lb_from_float<T>(v);
    }
}

// ---------------------------------------------------------------- the same norm and the token shift in one pass
// Block t makes h_t = norm(x_t) (written to `h`) and the mixer's input m_t = h_t + (prev - h_t) * mu, where prev is
// the norm of row t - 1 (made again here, so no block waits for another) or, for the first row of a request's
// portion, the request's state.  Both h_t and prev pass through the element type T first, so that a row blends
// with the same numbers whether its neighbour came in this step or in an earlier one.
template <typename T>
__global__ void rms_shift_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ w, const float* __restrict__ mu,
                                 T* __restrict__ h, int64_t ldh, T* __restrict__ m, int64_t ldm, T* __restrict__ state,
                                 const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots,
                                 int width, int groups, float eps) {
    extern __shared__ float inv_of[];          // [2][groups]
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, s = tok_seq[t], first = q_start[s], last = q_start[s + 1] - 1;
    const int part = width / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const float* cur = x + (size_t)t * ldx;
    const float* before = t > first ? x + (size_t)(t - 1) * ldx : nullptr;
    T* keep = state + (size_t)slots[s] * width;
    // Up to eight values a thread: its pieces of both rows, the gains and the state are asked for now, together with the sums' own
    // loads, instead of after the sums (one round trip to memory fewer; wider rows take the loads in the loop below).
    constexpr int kAhead = 8;
    const bool ahead = width <= kAhead * (int)blockDim.x;
    float a_cur[kAhead], a_prev[kAhead], a_w[kAhead], a_mu[kAhead];
    if (ahead) {
#pragma unroll
        for (int e = 0; e < kAhead; ++e) {
            const int i = threadIdx.x + e * blockDim.x;
            if (i < width) {
                a_cur[e] = cur[i];
                a_prev[e] = before != nullptr ? before[i] : lb_to_float(keep[i]);
                a_w[e] = w[i];
                a_mu[e] = mu[i];
            }
        }
    }
    // A warp per (row, group) sum: lanes stride over the part, then a shuffle tree; order fixed by the part's length.
    for (int job = warp; job < 2 * groups; job += n_warps) {
        const float* row = job < groups ? cur : before;
        if (row == nullptr) continue;
        const float* in = row + (size_t)(job % groups) * part;
        float ss = 0.0f;
        for (int i = lane; i < part; i += 32) ss = fmaf(in[i], in[i], ss);
        ss = lb_warp_sum(ss);
        if (lane == 0) inv_of[job] = 1.0f / sqrtf(ss / (float)part + eps);
    }
    __syncthreads();
    if (ahead) {
#pragma unroll
        for (int e = 0; e < kAhead; ++e) {
            const int i = threadIdx.x + e * blockDim.x;
            if (i >= width) break;
            const int g = i / part;
            const T hc = lb_from_float<T>(a_cur[e] * inv_of[g] * a_w[e]);
            const T hp = lb_from_float<T>(before != nullptr ? a_prev[e] * inv_of[groups + g] * a_w[e] : a_prev[e]);
            const float c = lb_to_float(hc), p = lb_to_float(hp);
            h[(size_t)t * ldh + i] = hc;
            m[(size_t)t * ldm + i] = lb_from_float<T>(c + (p - c) * a_mu[e]);
            if (first == last) keep[i] = hc;
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int g = i / part;
        const T hc = lb_from_float<T>(cur[i] * inv_of[g] * w[i]);
        const T hp = before != nullptr ? lb_from_float<T>(before[i] * inv_of[groups + g] * w[i]) : keep[i];
        const float c = lb_to_float(hc), p = lb_to_float(hp);
        h[(size_t)t * ldh + i] = hc;
        m[(size_t)t * ldm + i] = lb_from_float<T>(c + (p - c) * mu[i]);
        if (first == last) keep[i] = hc;       // a single token: this block read the state and may replace it
    }
}

// The token shift alone, from rows that are already normalised.
template <typename T>
__global__ void shift_kernel(const T* __restrict__ h, int64_t ldh, const float* __restrict__ mu, T* __restrict__ m, int64_t ldm,
                             T* __restrict__ state, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ q_start,
                             const int32_t* __restrict__ slots, int width) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, s = tok_seq[t], first = q_start[s], last = q_start[s + 1] - 1;
    T* keep = state + (size_t)slots[s] * width;
    const T* prev = t > first ? h + (size_t)(t - 1) * ldh : keep;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const T hc = h[(size_t)t * ldh + i];
        const float c = lb_to_float(hc), p = lb_to_float(prev[i]);
        m[(size_t)t * ldm + i] = lb_from_float<T>(c + (p - c) * mu[i]);
        if (first == last) keep[i] = hc;
    }
}

// The state of requests that brought more than one token: their last normalised row.  Runs after the shift, whose
// first-row blocks read the state.
template <typename T>
__global__ void shift_keep_kernel(const T* __restrict__ h, int64_t ldh, T* __restrict__ state, const int32_t* __restrict__ q_start,
                                  const int32_t* __restrict__ slots, int width) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int s = blockIdx.x, first = q_start[s], last = q_start[s + 1] - 1;
    if (last <= first) return;
    T* keep = state + (size_t)slots[s] * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) keep[i] = h[(size_t)last * ldh + i];
}

// ---------------------------------------------------------------- xIELU
// z > 0: a z^2 + z / 2;  z <= 0: b (exp(z) - 1 - z) + z / 2, with a = softplus(p) and b = 1/2 + softplus(q).
// (lb_softplus and lb_xielu of common.cuh: the same statements the products' epilogues use.)

// VEC: rows start on 16-byte boundaries and hold a multiple of a 16-byte piece; a thread takes four pieces, all asked for before any is
// used, the pieces of all rows numbered through.
template <typename T, bool VEC>
__global__ void xielu_kernel(T* __restrict__ z, int64_t ldz, int n_rows, int cols, const float* __restrict__ pq) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const float a = lb_softplus(pq[0]), b = 0.5f + lb_softplus(pq[1]);
    if (VEC) {
        constexpr int N = 16 / sizeof(T);
        const int per_row = cols / N;
        const long long total = (long long)n_rows * per_row, threads = (long long)gridDim.x * blockDim.x;
        const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
        uint4 raw[4];
        T* at[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long idx = first + k * threads;
            at[k] = nullptr;
            if (idx < total) {
                at[k] = z + (size_t)(idx / per_row) * ldz + (size_t)(idx % per_row) * N;
                raw[k] = *reinterpret_cast<const uint4*>(at[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (at[k] == nullptr) continue;
            T* v = reinterpret_cast<T*>(&raw[k]);
#pragma unroll
            for (int e = 0; e < N; ++e) v[e] = lb_from_float<T>(lb_xielu(lb_to_float(v[e]), a, b));
            *reinterpret_cast<uint4*>(at[k]) = raw[k];
        }
    } else {
        T* row = z + (size_t)blockIdx.x * ldz;
        for (int i = threadIdx.x + blockIdx.y * blockDim.x; i < cols; i += blockDim.x * gridDim.y) row[i] = lb_from_float<T>(lb_xielu(lb_to_float(row[i]), a, b));
    }
}

// ---------------------------------------------------------------- gated per-token side input
// g = gelu_tanh(G x) * e (e: the token's row of the side table), y = P g, x += y / sqrt(mean(y^2) + eps) * w, with G [dim, width]
// and P [width, dim]; the rows of x are 32-bit and stay so.  Two launches: the gate spread over (token, eight features) blocks, a warp
// per feature with lanes along the width; then a block per token, a thread per output column with P's short row in order.  Every sum's
// order depends on the sizes only.
template <typename T>
__global__ void __launch_bounds__(256)
side_gate_kernel(const float* __restrict__ x, int64_t ldx, const int32_t* __restrict__ tokens, const T* __restrict__ table, const T* __restrict__ G,
                 float* __restrict__ g, int width, int dim) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, d = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (d >= dim) return;
    const T* row = G + (size_t)d * width;
    const float* xr = x + (size_t)t * ldx;
    const float e = lb_to_float(table[(size_t)tokens[t] * dim + d]);        // asked for under the sum, not after it
    float acc = 0.0f;
    for (int c = lane; c < width; c += 32) acc = fmaf(lb_to_float(row[c]), xr[c], acc);
    acc = lb_warp_sum(acc);
    if (lane == 0) g[(size_t)t * dim + d] = lb_gelu_tanh(acc) * e;
}

template <typename T>
__global__ void __launch_bounds__(256)
side_proj_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ g, const T* __restrict__ P, const float* __restrict__ w, int width, int dim,
                 float eps) {
    extern __shared__ float sm[];              // g [dim], then y [width]
    __shared__ float scratch[33];
    float* gs = sm;
    float* ys = sm + dim;
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) gs[d] = g[(size_t)t * dim + d];
    __syncthreads();
    float ss = 0.0f;
    constexpr int N = 16 / sizeof(T);
    const bool pieces = dim % N == 0 && (reinterpret_cast<uintptr_t>(P) & 15) == 0;        // P's rows start on 16-byte boundaries
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const T* row = P + (size_t)c * dim;
        float acc = 0.0f;
        if (pieces) {
            for (int d = 0; d < dim; d += N) {
                const uint4 raw = *reinterpret_cast<const uint4*>(row + d);
                const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int k = 0; k < N; ++k) acc = fmaf(lb_to_float(v[k]), gs[d + k], acc);      // the same order as one by one
            }
        } else {
            for (int d = 0; d < dim; ++d) acc = fmaf(lb_to_float(row[d]), gs[d], acc);
        }
        ys[c] = acc;
        ss = fmaf(acc, acc, ss);
    }
    // The row to add to and its gains: asked for before the block's sum (up to eight values a thread), not after it.
    float* xr = x + (size_t)t * ldx;
    constexpr int kAhead = 8;
    const bool ahead = width <= kAhead * (int)blockDim.x;
    float a_x[kAhead], a_w[kAhead];
    if (ahead) {
#pragma unroll
        for (int e = 0; e < kAhead; ++e) {
            const int c = threadIdx.x + e * blockDim.x;
            if (c < width) {
                a_x[e] = xr[c];
                a_w[e] = w[c];
            }
        }
    }
    const float inv = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)width + eps);
    if (ahead) {
#pragma unroll
        for (int e = 0; e < kAhead; ++e) {
            const int c = threadIdx.x + e * blockDim.x;
            if (c < width) xr[c] = a_x[e] + ys[c] * inv * a_w[e];
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) xr[c] += ys[c] * inv * w[c];
}

// The pieces around two library products for steps of many tokens (bfloat16).
__global__ void rows_to_bf16_kernel(const float* __restrict__ x, int64_t ldx, __nv_bfloat16* __restrict__ y, int64_t ldy, int cols) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const float* in = x + (size_t)blockIdx.x * ldx;
    __nv_bfloat16* out = y + (size_t)blockIdx.x * ldy;
    if (cols % 4 == 0 && ldx % 4 == 0 && ldy % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
        for (int i = threadIdx.x * 4; i < cols; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(in + i);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            *reinterpret_cast<uint2*>(out + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
        return;
    }
    for (int i = threadIdx.x; i < cols; i += blockDim.x) out[i] = __float2bfloat16_rn(in[i]);
}

__global__ void side_gate_finish_kernel(const float* __restrict__ pre, int64_t ldp, const int32_t* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                                        __nv_bfloat16* __restrict__ g16, int64_t ldg, int dim) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < dim; d += blockDim.x)
        g16[(size_t)t * ldg + d] = __float2bfloat16_rn(lb_gelu_tanh(pre[(size_t)t * ldp + d]) * __bfloat162float(table[(size_t)tokens[t] * dim + d]));
}

__global__ void rms_add_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ y, int64_t ldy, const float* __restrict__ w, int width, float eps) {
    __shared__ float scratch[33];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const float* yr = y + (size_t)blockIdx.x * ldy;
    float* xr = x + (size_t)blockIdx.x * ldx;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
    const float inv = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) xr[i] += yr[i] * inv * w[i];
}

template <typename T>
int launch_token_side(float* x, int64_t ldx, const int32_t* tokens, const void* table, const void* G, const void* P, const float* w, float* g,
                      int n_tokens, int width, int dim, float eps, cudaStream_t s) {
    const size_t smem = (size_t)(width + dim) * sizeof(float);
    if (smem > 200 * 1024) return lb_fail(LB_ERR_UNSUPPORTED, "token side input: rows of %d values with %d gate features do not fit a block", width, dim);
    if (smem > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(side_proj_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LB_CHECK_CUDA(lb_launch_overlapped(side_gate_kernel<T>, dim3(n_tokens, (dim + 7) / 8), dim3(256), 0, s, (const float*)x, ldx, tokens, (const T*)table,
                                       (const T*)G, g, width, dim));
    LB_CHECK_CUDA(lb_launch_overlapped(side_proj_kernel<T>, dim3(n_tokens), dim3(256), smem, s, x, ldx, (const float*)g, (const T*)P, w, width, dim, eps));
    return LB_OK;
}

}  // namespace

extern "C" int lb_rms_groups(int out_dtype, const float* x, int64_t ldx, const int32_t* rows, const float* weight, void* y, int64_t ldy,
                             int n_rows, int width, int groups, float eps, void* stream) {
    return lb_rms_groups_offset(out_dtype, x, ldx, rows, weight, 0.0f, y, ldy, n_rows, width, groups, eps, stream);
}

extern "C" int lb_rms_groups_offset(int out_dtype, const float* x, int64_t ldx, const int32_t* rows, const float* weight, float gain_offset, void* y,
                                    int64_t ldy, int n_rows, int width, int groups, float eps, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0 && groups > 0 && width % groups == 0, "rms norm: %d values do not split into %d equal groups", width, groups);
    if (n_rows == 0) return LB_OK;
    const int part = width / groups, threads = part >= 1024 ? 256 : part >= 256 ? 128 : part > 32 ? 64 : 32;
    auto s = static_cast<cudaStream_t>(stream);
    if (out_dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(rms_groups_kernel<float>, dim3(n_rows, groups), dim3(threads), 0, s, x, ldx, rows, weight, (float*)y, ldy, part, eps, gain_offset));
    else if (out_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(rms_groups_kernel<__nv_bfloat16>, dim3(n_rows, groups), dim3(threads), 0, s, x, ldx, rows, weight,
                                           (__nv_bfloat16*)y, ldy, part, eps, gain_offset));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "rms norm: unknown dtype %d", out_dtype);
    return LB_OK;
}

extern "C" int lb_rms_shift(int dtype, const float* x, int64_t ldx, const float* weight, const float* mix, void* h, int64_t ldh, void* m,
                            int64_t ldm, void* state, const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots, int n_tokens,
                            int n_seq, int decode_only, int width, int groups, float eps, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && width > 0 && groups > 0 && width % groups == 0, "rms norm: %d values do not split into %d equal groups", width, groups);
    LB_CHECK_ARG(groups <= 4096, "rms norm: %d groups are more than a block keeps", groups);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const int threads = width >= 1024 ? 256 : 128;
    const size_t smem = 2 * (size_t)groups * sizeof(float);
    if (dtype == LB_F32) {
        LB_CHECK_CUDA(lb_launch_overlapped(rms_shift_kernel<float>, dim3(n_tokens), dim3(threads), smem, s, x, ldx, weight, mix, (float*)h, ldh, (float*)m,
                                           ldm, (float*)state, tok_seq, q_start, slots, width, groups, eps));
        if (!decode_only)
            LB_CHECK_CUDA(lb_launch_overlapped(shift_keep_kernel<float>, dim3(n_seq), dim3(threads), 0, s, (const float*)h, ldh, (float*)state, q_start, slots, width));
    } else if (dtype == LB_BF16) {
        using B = __nv_bfloat16;
        LB_CHECK_CUDA(lb_launch_overlapped(rms_shift_kernel<B>, dim3(n_tokens), dim3(threads), smem, s, x, ldx, weight, mix, (B*)h, ldh, (B*)m, ldm,
                                           (B*)state, tok_seq, q_start, slots, width, groups, eps));
        if (!decode_only)
            LB_CHECK_CUDA(lb_launch_overlapped(shift_keep_kernel<B>, dim3(n_seq), dim3(threads), 0, s, (const B*)h, ldh, (B*)state, q_start, slots, width));
    } else return lb_fail(LB_ERR_INVALID_ARGUMENT, "token shift: unknown dtype %d", dtype);
    return LB_OK;
}

extern "C" int lb_token_shift(int dtype, const void* h, int64_t ldh, const float* mix, void* m, int64_t ldm, void* state,
                              const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots, int n_tokens, int n_seq, int decode_only,
                              int width, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && width > 0, "token shift: bad sizes n_tokens=%d width=%d", n_tokens, width);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == LB_F32) {
        LB_CHECK_CUDA(lb_launch_overlapped(shift_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)h, ldh, mix, (float*)m, ldm, (float*)state,
                                           tok_seq, q_start, slots, width));
        if (!decode_only)
            LB_CHECK_CUDA(lb_launch_overlapped(shift_keep_kernel<float>, dim3(n_seq), dim3(threads), 0, s, (const float*)h, ldh, (float*)state, q_start, slots, width));
    } else if (dtype == LB_BF16) {
        using B = __nv_bfloat16;
        LB_CHECK_CUDA(lb_launch_overlapped(shift_kernel<B>, dim3(n_tokens), dim3(threads), 0, s, (const B*)h, ldh, mix, (B*)m, ldm, (B*)state, tok_seq,
                                           q_start, slots, width));
        if (!decode_only)
            LB_CHECK_CUDA(lb_launch_overlapped(shift_keep_kernel<B>, dim3(n_seq), dim3(threads), 0, s, (const B*)h, ldh, (B*)state, q_start, slots, width));
    } else return lb_fail(LB_ERR_INVALID_ARGUMENT, "token shift: unknown dtype %d", dtype);
    return LB_OK;
}

extern "C" int lb_xielu(int dtype, void* z, int64_t ldz, int n_rows, int cols, const float* pq, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && cols > 0 && pq != nullptr, "xielu: bad sizes n_rows=%d cols=%d", n_rows, cols);
    if (n_rows == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const int piece = dtype == LB_F32 ? 4 : 8;
    const bool vec = cols % piece == 0 && ldz % piece == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0;
    const long long pieces = (long long)n_rows * (cols / piece);
    const dim3 grid = vec ? dim3((unsigned)((pieces + 1023) / 1024)) : dim3(n_rows, (cols + 2047) / 2048);
    if (dtype == LB_F32) {
        if (vec) LB_CHECK_CUDA(lb_launch_overlapped(xielu_kernel<float, true>, grid, dim3(256), 0, s, (float*)z, ldz, n_rows, cols, pq));
        else LB_CHECK_CUDA(lb_launch_overlapped(xielu_kernel<float, false>, grid, dim3(256), 0, s, (float*)z, ldz, n_rows, cols, pq));
    } else if (dtype == LB_BF16) {
        if (vec) LB_CHECK_CUDA(lb_launch_overlapped(xielu_kernel<__nv_bfloat16, true>, grid, dim3(256), 0, s, (__nv_bfloat16*)z, ldz, n_rows, cols, pq));
        else LB_CHECK_CUDA(lb_launch_overlapped(xielu_kernel<__nv_bfloat16, false>, grid, dim3(256), 0, s, (__nv_bfloat16*)z, ldz, n_rows, cols, pq));
    } else return lb_fail(LB_ERR_INVALID_ARGUMENT, "xielu: unknown dtype %d", dtype);
    return LB_OK;
}

extern "C" int lb_token_side(int dtype, float* x, int64_t ldx, const int32_t* tokens, const void* table, const void* gate, const void* proj,
                             const float* weight, float* g, int n_tokens, int width, int dim, float eps, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && width > 0 && dim > 0 && g != nullptr, "token side input: bad sizes n_tokens=%d width=%d dim=%d", n_tokens, width, dim);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (dtype == LB_F32) return launch_token_side<float>(x, ldx, tokens, table, gate, proj, weight, g, n_tokens, width, dim, eps, s);
    if (dtype == LB_BF16) return launch_token_side<__nv_bfloat16>(x, ldx, tokens, table, gate, proj, weight, g, n_tokens, width, dim, eps, s);
    return lb_fail(LB_ERR_INVALID_ARGUMENT, "token side input: unknown dtype %d", dtype);
}

extern "C" int lb_rows_to_bf16(const float* x, int64_t ldx, void* y, int64_t ldy, int n_rows, int cols, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && cols > 0, "rows to bfloat16: bad sizes rows=%d cols=%d", n_rows, cols);
    if (n_rows == 0) return LB_OK;
    LB_CHECK_CUDA(lb_launch_overlapped(rows_to_bf16_kernel, dim3(n_rows), dim3(256), 0, static_cast<cudaStream_t>(stream), x, ldx, (__nv_bfloat16*)y, ldy, cols));
    return LB_OK;
}

extern "C" int lb_side_gate_finish(const float* pre, int64_t ldp, const int32_t* tokens, const void* table, void* g16, int64_t ldg, int n_tokens, int dim,
                                   void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && dim > 0, "token side input: bad sizes n_tokens=%d dim=%d", n_tokens, dim);
    if (n_tokens == 0) return LB_OK;
    LB_CHECK_CUDA(lb_launch_overlapped(side_gate_finish_kernel, dim3(n_tokens), dim3(dim >= 256 ? 256 : dim > 64 ? 128 : 64), 0, static_cast<cudaStream_t>(stream), pre,
                                       ldp, tokens, (const __nv_bfloat16*)table, (__nv_bfloat16*)g16, ldg, dim));
    return LB_OK;
}

extern "C" int lb_rms_add(float* x, int64_t ldx, const float* y, int64_t ldy, const float* weight, int n_rows, int width, float eps, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0, "rms add: bad sizes rows=%d width=%d", n_rows, width);
    if (n_rows == 0) return LB_OK;
    LB_CHECK_CUDA(lb_launch_overlapped(rms_add_kernel, dim3(n_rows), dim3(256), 0, static_cast<cudaStream_t>(stream), x, ldx, y, ldy, weight, width, eps));
    return LB_OK;
}
