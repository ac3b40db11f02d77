// Recurrences with a matrix of state per head, and the short causal convolution in front of one.
//
// Both mixers built on this file keep, per request and head, a float32 matrix S [N, dv] and step
//     S <- a_t S + k_t (s_t v_t)^T          y_t = S^T q_t + c v_t
// token by token:
//   decayed linear attention   a_t = decay_h (a constant of the head), k, q, v = silu of the projection,
//                              s_t = 1, c = 0, N = key size;
//   selective scan (SSD)       a_t = exp(-exp(A_log_h) dt_t), dt_t = softplus(dt + bias_h), k_t = B_t,
//                              q_t = C_t (shared by the heads of a group), v_t = x_t, s_t = dt_t, c = D_h.
// One thread owns one column of S (its N elements in registers) for the tokens that one request
// brings in this step; the per-token vectors k and q reach the threads through shared memory in tiles
// of 16 tokens.  The state is read from the request's slot before the first token and written back
// after the last, so a prompt may arrive in any portions; a slot is zeroed by the cache at admission.
// Everything but the loads of bfloat16 projections is float32.
#include "common.cuh"

namespace b200 {

constexpr int kScanTile = 16;       // tokens staged at a time
constexpr int kScanColumns = 64;    // columns of S per block

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

struct ScanParams {
    // common
    const int* query_start;     // [R + 1]
    const int* slots;           // [R]
    float* state;               // [slots + 1, H, N, dv]
    float* y;                   // [T, H * dv]
    int heads, n, dv;
    // linear attention: packed projection rows [q | k | v] of `stride` elements
    const void* proj;
    int stride, off_q, off_k, off_v;
    const float* decay;         // [H]
    // selective scan: xbc float32 [T, xbc_width] = [x | B | C], dt from the projection
    const float* xbc;
    int xbc_width, off_b, off_c, group_heads;   // heads per group
    int off_dt;                 // column of dt in `proj`
    const float* dt_bias;       // [H]
    const float* a_log;         // [H]
    const float* skip;          // [H]
};

template <typename T, int NMAX, bool SSD>
__global__ void __launch_bounds__(kScanColumns) recurrence_kernel(ScanParams p) {
    __shared__ __align__(16) float k_s[kScanTile][NMAX];
    __shared__ __align__(16) float q_s[kScanTile][NMAX];
    __shared__ float a_s[kScanTile], s_s[kScanTile];
    const int request = blockIdx.x, head = blockIdx.y;
    const int column = blockIdx.z * kScanColumns + threadIdx.x;
    const bool live = column < p.dv;
    const int begin = p.query_start[request], end = p.query_start[request + 1];
    if (begin >= end) return;
    const int n = p.n, n4 = (p.n + 3) & ~3;
    float* state = p.state + (((size_t)p.slots[request] * p.heads + head) * n) * p.dv + column;
    float S[NMAX];
#pragma unroll
    for (int i = 0; i < NMAX; ++i) S[i] = (live && i < n) ? state[(size_t)i * p.dv] : 0.0f;
    const T* proj = (const T*)p.proj;
    const float decay = SSD ? 0.0f : p.decay[head];
    const float skip = SSD ? p.skip[head] : 0.0f;
    const float a_neg = SSD ? -expf(p.a_log[head]) : 0.0f;
    const float dt_bias = SSD ? p.dt_bias[head] : 0.0f;
    const int group = SSD ? head / p.group_heads : 0;

    for (int t0 = begin; t0 < end; t0 += kScanTile) {
        const int count = min(kScanTile, end - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < count * n4; idx += blockDim.x) {
            const int t = idx / n4, i = idx - t * n4;
            const size_t token = (size_t)(t0 + t);
            if (i >= n) {           // the tail of the last group of four: zeros keep S[i] at zero
                k_s[t][i] = q_s[t][i] = 0.0f;
            } else if (SSD) {
                const float* row = p.xbc + token * p.xbc_width;
                k_s[t][i] = row[p.off_b + group * n + i];
                q_s[t][i] = row[p.off_c + group * n + i];
            } else {
                const T* row = proj + token * p.stride;
                k_s[t][i] = silu_f(to_float(row[p.off_k + head * n + i]));
                q_s[t][i] = silu_f(to_float(row[p.off_q + head * n + i]));
            }
        }
        if (threadIdx.x < count) {
            if (SSD) {
                const float dt = softplus_f(to_float(proj[(size_t)(t0 + threadIdx.x) * p.stride + p.off_dt + head]) + dt_bias);
                a_s[threadIdx.x] = expf(a_neg * dt);
                s_s[threadIdx.x] = dt;
            } else {
                a_s[threadIdx.x] = decay;
                s_s[threadIdx.x] = 1.0f;
            }
        }
        __syncthreads();
        if (!live) continue;
        for (int t = 0; t < count; ++t) {
            const size_t token = (size_t)(t0 + t);
            float v;
            if (SSD) v = p.xbc[token * p.xbc_width + head * p.dv + column];
            else v = silu_f(to_float(proj[token * p.stride + p.off_v + head * p.dv + column]));
            const float a = a_s[t], sv = s_s[t] * v;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NMAX; i += 4) {
                if (i < n) {        // a group of four that reaches past n meets zeros there
                    const float4 k4 = *reinterpret_cast<const float4*>(&k_s[t][i]);
                    const float4 q4 = *reinterpret_cast<const float4*>(&q_s[t][i]);
                    S[i] = fmaf(a, S[i], k4.x * sv);
                    S[i + 1] = fmaf(a, S[i + 1], k4.y * sv);
                    S[i + 2] = fmaf(a, S[i + 2], k4.z * sv);
                    S[i + 3] = fmaf(a, S[i + 3], k4.w * sv);
                    acc = fmaf(S[i], q4.x, acc);
                    acc = fmaf(S[i + 1], q4.y, acc);
                    acc = fmaf(S[i + 2], q4.z, acc);
                    acc = fmaf(S[i + 3], q4.w, acc);
                }
            }
            p.y[token * ((size_t)p.heads * p.dv) + head * p.dv + column] = fmaf(skip, v, acc);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NMAX; ++i)
            if (i < n) state[(size_t)i * p.dv] = S[i];
    }
}

template <typename T, bool SSD>
int launch_recurrence(const ScanParams& p, int requests, cudaStream_t stream) {
    dim3 grid(requests, p.heads, (p.dv + kScanColumns - 1) / kScanColumns);
    if (p.heads > 65535) return fail("recurrence", "more than 65535 heads");
    if (p.n <= 32) recurrence_kernel<T, 32, SSD><<<grid, kScanColumns, 0, stream>>>(p);
    else if (p.n <= 64) recurrence_kernel<T, 64, SSD><<<grid, kScanColumns, 0, stream>>>(p);
    else if (p.n <= 128) recurrence_kernel<T, 128, SSD><<<grid, kScanColumns, 0, stream>>>(p);
    else if (p.n <= 256) recurrence_kernel<T, 256, SSD><<<grid, kScanColumns, 0, stream>>>(p);
    else return fail("recurrence", "a state of more than 256 rows per head is not built");
    return check_launch("recurrence");
}

// out[t, c] = silu(bias[c] + sum_i w[c, i] * in[t - (taps - 1 - i), c]) within one request; inputs
// before the step's portion come from the request's state (its last taps - 1 inputs, oldest first,
// zeros before the sequence's start).
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int stride, int offset, const float* __restrict__ w,
                                        const float* __restrict__ bias, const float* __restrict__ state,
                                        const int* __restrict__ token_request, const int* __restrict__ query_start,
                                        const int* __restrict__ slots, float* __restrict__ out, int channels, int taps) {
    const int token = blockIdx.x;
    const int request = token_request[token];
    const int place = token - query_start[request];        // index within this step's portion
    const float* kept = state + (size_t)slots[request] * (taps - 1) * channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float acc = bias[c];
        for (int i = 0; i < taps; ++i) {
            const int back = taps - 1 - i;
            float v;
            if (place - back >= 0) v = to_float(in[(size_t)(token - back) * stride + offset + c]);
            else v = kept[(size_t)(taps - 1 + place - back) * channels + c];
            acc = fmaf(w[(size_t)c * taps + i], v, acc);
        }
        out[(size_t)token * channels + c] = silu_f(acc);
    }
}

// After the convolution: the request's last taps - 1 inputs, oldest first.  One thread per request
// and channel reads what it keeps of the old state before it writes.
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ in, int stride, int offset, float* __restrict__ state,
                                  const int* __restrict__ query_start, const int* __restrict__ slots, int channels,
                                  int taps) {
    constexpr int kMost = 15;
    const int request = blockIdx.x;
    const int begin = query_start[request], length = query_start[request + 1] - begin;
    if (length <= 0) return;
    float* kept = state + (size_t)slots[request] * (taps - 1) * channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float fresh[kMost];
#pragma unroll
        for (int i = 0; i < kMost; ++i) {
            if (i < taps - 1) {
                const int place = length - (taps - 1) + i;
                fresh[i] = place >= 0 ? to_float(in[(size_t)(begin + place) * stride + offset + c])
                                      : kept[(size_t)(i + length) * channels + c];
            }
        }
#pragma unroll
        for (int i = 0; i < kMost; ++i)
            if (i < taps - 1) kept[(size_t)i * channels + c] = fresh[i];
    }
}

}  // namespace b200

// Decayed linear attention over the packed projection `proj` [T, stride] = [.. q .. k .. v ..] (columns
// off_q, off_k, off_v; q and k are heads x n, v heads x dv; silu is applied on load).  y: float32
// [T, heads * dv].  state: float32 [slots + 1, heads, n, dv].  dtype of proj: 0 float32, 1 bfloat16.
B200_EXPORT int b200_decayed_linear_attention(const void* proj, int stride, int off_q, int off_k, int off_v,
                                              const float* decay, const int* query_start, const int* slots,
                                              float* state, float* y, int requests, int heads, int n, int dv,
                                              int dtype, cudaStream_t stream) {
    using namespace b200;
    if (requests == 0) return 0;
    ScanParams p = {};
    p.query_start = query_start; p.slots = slots; p.state = state; p.y = y;
    p.heads = heads; p.n = n; p.dv = dv;
    p.proj = proj; p.stride = stride; p.off_q = off_q; p.off_k = off_k; p.off_v = off_v; p.decay = decay;
    if (dtype == 0) return launch_recurrence<float, false>(p, requests, stream);
    if (dtype == 1) return launch_recurrence<__nv_bfloat16, false>(p, requests, stream);
    return fail("decayed_linear_attention", "dtype must be 0 (float32) or 1 (bfloat16)");
}

// Selective scan.  xbc: float32 [T, xbc_width] = [x: heads * dv | B: groups * n | C: groups * n]
// (after the convolution and silu); dt: column off_dt + head of `proj` [T, stride]; y float32
// [T, heads * dv]; state float32 [slots + 1, heads, n, dv].
B200_EXPORT int b200_selective_scan(const float* xbc, int xbc_width, const void* proj, int stride, int off_dt,
                                    const float* dt_bias, const float* a_log, const float* skip,
                                    const int* query_start, const int* slots, float* state, float* y,
                                    int requests, int heads, int groups, int n, int dv, int dtype,
                                    cudaStream_t stream) {
    using namespace b200;
    if (requests == 0) return 0;
    if (groups <= 0 || heads % groups) return fail("selective_scan", "heads must be a multiple of groups");
    ScanParams p = {};
    p.query_start = query_start; p.slots = slots; p.state = state; p.y = y;
    p.heads = heads; p.n = n; p.dv = dv;
    p.proj = proj; p.stride = stride; p.off_dt = off_dt;
    p.xbc = xbc; p.xbc_width = xbc_width; p.off_b = heads * dv; p.off_c = heads * dv + groups * n;
    p.group_heads = heads / groups;
    p.dt_bias = dt_bias; p.a_log = a_log; p.skip = skip;
    if (dtype == 0) return launch_recurrence<float, true>(p, requests, stream);
    if (dtype == 1) return launch_recurrence<__nv_bfloat16, true>(p, requests, stream);
    return fail("selective_scan", "dtype must be 0 (float32) or 1 (bfloat16)");
}

// The convolution reads the state, the second kernel replaces it: call them in this order.
// in: [T, stride] with the channels at column `offset`; w float32 [channels, taps] (last column: the
// current token); state float32 [slots + 1, taps - 1, channels]; out float32 [T, channels].
B200_EXPORT int b200_causal_conv_silu(const void* in, int stride, int offset, const float* w, const float* bias,
                                      float* state, const int* token_request, const int* query_start,
                                      const int* slots, float* out, int tokens, int requests, int channels, int taps,
                                      int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0) return 0;
    if (taps < 1 || taps > 16) return fail("causal_conv_silu", "1 to 16 taps are built");
    if (dtype != 0 && dtype != 1) return fail("causal_conv_silu", "dtype must be 0 (float32) or 1 (bfloat16)");
    const int threads = 128;
    const int tiles = min((channels + threads - 1) / threads, 65535);
    if (dtype == 0)
        causal_conv_silu_kernel<float><<<dim3(tokens, tiles), threads, 0, stream>>>(
            (const float*)in, stride, offset, w, bias, state, token_request, query_start, slots, out, channels, taps);
    else
        causal_conv_silu_kernel<__nv_bfloat16><<<dim3(tokens, tiles), threads, 0, stream>>>(
            (const __nv_bfloat16*)in, stride, offset, w, bias, state, token_request, query_start, slots, out, channels, taps);
    if (int status = check_launch("causal_conv_silu")) return status;
    if (taps == 1) return 0;
    if (dtype == 0)
        conv_state_kernel<float><<<dim3(requests, tiles), threads, 0, stream>>>(
            (const float*)in, stride, offset, state, query_start, slots, channels, taps);
    else
        conv_state_kernel<__nv_bfloat16><<<dim3(requests, tiles), threads, 0, stream>>>(
            (const __nv_bfloat16*)in, stride, offset, state, query_start, slots, channels, taps);
    return check_launch("conv_state");
}
