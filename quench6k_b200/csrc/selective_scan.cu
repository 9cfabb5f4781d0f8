// The recurrent half of a selective state-space mixer (Mamba, first form), for any mix of prompt
// portions and single tokens, with the state of every request in its slot:
//
//   conv:  u[t, c] = silu(bias[c] + sum_k w[c, k] * x[t - (taps-1-k), c])      inputs before the portion come from the slot's
//                                                                              tail of the last taps-1 inputs, zeros at the start
//   scan:  dt = softplus(dt_raw[t, c] + dt_bias[c])
//          S[c, n] <- exp(dt * A[c, n]) * S[c, n] + dt * u[t, c] * B[t, n]
//          y[t, c] = (sum_n S[c, n] * C[t, n] + D[c] * u[t, c]) * silu(z[t, c])
//
// The state S, dt, the decay and every sum of the recurrence are FP32; u leaves the convolution in
// the operand dtype (it is the next product's input) and enters the recurrence as stored.  A group of
// L lanes owns a channel (state index n = lane + L * k); the sum over n is a butterfly over those
// lanes, so its order depends on nothing but N.  Tokens of a request are walked in order, so a prompt
// cut anywhere leaves the same state as the whole prompt.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;
constexpr int SCAN_TILE = 16;      // tokens whose B and C rows are staged in shared memory at a time
constexpr int MAX_PER_LANE = 8;    // states per lane

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// grid (T, ceil(C / 256)); x: FP32 [T, ldx] (first C columns); tail: FP32 [slots, taps-1, C].
template <typename T>
__global__ void __launch_bounds__(256) conv_silu_kernel(const float* x, int ldx, const float* w, const float* bias, const float* tail,
                                                        const int* req_of_token, const int* q_start, const int* slot_ids, T* out,
                                                        int C, int taps) {
    pdl_enter();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r = req_of_token[t], first = q_start[r], i = t - first;
    const float* old = tail + (size_t)slot_ids[r] * (taps - 1) * C;
    float acc = bias[c];
    for (int k = 0; k < taps; ++k) {
        const int j = i - (taps - 1 - k);                        // index within the portion; negative: before it
        const float v = j >= 0 ? x[(size_t)(first + j) * ldx + c] : old[(size_t)(taps - 1 + j) * C + c];
        acc = fmaf(w[(size_t)c * taps + k], v, acc);
    }
    out[(size_t)t * C + c] = from_f32<T>(silu_f(acc));
}

// grid (R, ceil(C / (128 / L))), 128 threads; dynamic shared memory 2 * SCAN_TILE * N floats.
template <typename T>
__global__ void __launch_bounds__(128) selective_scan_kernel(const T* u, const float* dt_raw, const float* dt_bias, const float* proj, int ldp,
                                                             int b_col, int c_col, const float* A, const float* Dskip, const float* xz,
                                                             int ldx, int z_col, float* state, float* tail, const int* q_start,
                                                             const int* slot_ids, T* out, int C, int N, int L, int taps) {
    pdl_enter();
    extern __shared__ float bc[];              // [SCAN_TILE][N] of B, then the same of C
    const int r = blockIdx.x;
    const int per_block = blockDim.x / L;
    const int c = blockIdx.y * per_block + threadIdx.x / L, sub = threadIdx.x % L;
    const bool live = c < C;
    const int first = q_start[r], n_tok = q_start[r + 1] - first, slot = slot_ids[r];
    float S[MAX_PER_LANE], a[MAX_PER_LANE];
    float* Sg = state + ((size_t)slot * C + (live ? c : 0)) * N;
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
        const int n = sub + L * k;
        const bool has = live && n < N;
        S[k] = has ? Sg[n] : 0.0f;
        a[k] = has ? A[(size_t)c * N + n] : 0.0f;
    }
    const float bias = live ? dt_bias[c] : 0.0f, dskip = live ? Dskip[c] : 0.0f;
    for (int t0 = 0; t0 < n_tok; t0 += SCAN_TILE) {
        const int nt = min(SCAN_TILE, n_tok - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
            const int tt = i / N, n = i % N;
            const float* pr = proj + (size_t)(first + t0 + tt) * ldp;
            bc[i] = pr[b_col + n];
            bc[SCAN_TILE * N + i] = pr[c_col + n];
        }
        __syncthreads();
        float dtv[SCAN_TILE], uv[SCAN_TILE];
#pragma unroll
        for (int tt = 0; tt < SCAN_TILE; ++tt) {                 // nothing here waits for the recurrence
            const bool has = live && tt < nt;
            const size_t row = (size_t)(first + t0 + (has ? tt : 0));
            dtv[tt] = has ? softplus_f(dt_raw[row * C + c] + bias) : 0.0f;
            uv[tt] = has ? to_f32(u[row * C + c]) : 0.0f;
        }
#pragma unroll
        for (int tt = 0; tt < SCAN_TILE; ++tt) {
            if (tt < nt) {
                const float dt = dtv[tt], du = dtv[tt] * uv[tt];
                const float* Bt = bc + tt * N;
                const float* Ct = bc + SCAN_TILE * N + tt * N;
                float y = 0.0f;
#pragma unroll
                for (int k = 0; k < MAX_PER_LANE; ++k) {
                    const int n = sub + L * k;
                    if (n < N) {
                        // exp(dt A) S as S + expm1(dt A) S: a decay close to 1 keeps its distance from 1 to full precision, so
                        // that no rounding of the factor itself (always the same way for a given dt A) adds up over a long context
                        S[k] = fmaf(expm1f(dt * a[k]), S[k], S[k]) + du * Bt[n];
                        y = fmaf(S[k], Ct[n], y);
                    }
                }
                for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (live && sub == 0) {
                    const size_t row = (size_t)(first + t0 + tt);
                    const float z = xz[row * ldx + z_col + c];
                    out[row * C + c] = from_f32<T>(fmaf(dskip, uv[tt], y) * silu_f(z));
                }
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
        const int n = sub + L * k;
        if (n < N) Sg[n] = S[k];
    }
    if (sub == 0 && taps > 1) {
        // the last taps-1 inputs of the convolution: the end of this portion, preceded by what is left of the old tail
        float* tl = tail + (size_t)slot * (taps - 1) * C + c;
        float keep[MAX_TAPS];
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) {
            if (j < taps - 1) {
                const int src = n_tok - (taps - 1) + j;          // index within the portion
                keep[j] = src >= 0 ? xz[(size_t)(first + src) * ldx + c] : tl[(size_t)(j + n_tok) * C];
            }
        }
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j)
            if (j < taps - 1) tl[(size_t)j * C] = keep[j];
    }
}

template <typename T>
__global__ void cast_columns_kernel(const float* src, int ld, int col0, int n, T* out, size_t total) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    out[i] = from_f32<T>(src[(i / n) * ld + col0 + i % n]);
}

}  // namespace

// out[t, c] = dtype(silu(causal convolution over the request's inputs)).  x: FP32 [T, ldx], channels in its first C columns.
// w: FP32 [C, taps] (last column: the current token's), bias FP32 [C], tail FP32 [slots, taps-1, C] (read only here; the scan
// kernel moves it on).
Q6K_API int q6k_conv_silu(const float* x, int ldx, const float* w, const float* bias, const float* tail, const int* req_of_token,
                          const int* q_start, const int* slot_ids, void* out, int T_, int C, int taps, int dtype, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && C > 0 && taps >= 1 && taps <= MAX_TAPS, "conv_silu: bad sizes T=%d C=%d taps=%d (at most %d taps)", T_, C, taps, MAX_TAPS);
    dim3 grid(T_, (C + 255) / 256);
    Q6K_REQUIRE(grid.y <= 65535, "conv_silu: %d channels exceed the grid limit", C);
    Q6K_DISPATCH(dtype, q6k_launch(conv_silu_kernel<T>, grid, 256, 0, st, x, ldx, w, bias, tail, req_of_token, q_start, slot_ids,
                                   (T*)out, C, taps););
    return q6k_check_launch("conv_silu");
}

// How many lanes share a channel for N states: the power of two that leaves each lane about four.
Q6K_API int q6k_selective_scan_lanes(int N) {
    int L = 1;
    while (L < 32 && L * 4 < N) L *= 2;
    return L;
}

// u: dtype [T, C] (the convolution's result); dt_raw: FP32 [T, C]; proj: FP32 [T, ldp] with B in columns b_col.. and C in
// c_col.. (N each); A: FP32 [C, N] (negative); Dskip: FP32 [C]; xz: FP32 [T, ldx] with the convolution's inputs in columns
// 0.. and the gate z in columns z_col..; state: FP32 [slots, C, N]; tail: FP32 [slots, taps-1, C]; out: dtype [T, C].
Q6K_API int q6k_selective_scan(const void* u, const float* dt_raw, const float* dt_bias, const float* proj, int ldp, int b_col, int c_col,
                               const float* A, const float* Dskip, const float* xz, int ldx, int z_col, float* state, float* tail,
                               const int* q_start, const int* slot_ids, void* out, int R, int C, int N, int taps, int dtype,
                               cudaStream_t st) {
    if (R == 0) return 0;
    const int L = q6k_selective_scan_lanes(N);
    Q6K_REQUIRE(R > 0 && C > 0 && N > 0 && N <= L * MAX_PER_LANE, "selective_scan: bad sizes R=%d C=%d N=%d (at most %d states)", R, C, N,
                32 * MAX_PER_LANE);
    Q6K_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "selective_scan: %d taps (at most %d)", taps, MAX_TAPS);
    const int per_block = 128 / L;
    dim3 grid(R, (C + per_block - 1) / per_block);
    Q6K_REQUIRE(grid.y <= 65535, "selective_scan: %d channels exceed the grid limit", C);
    const size_t smem = (size_t)2 * SCAN_TILE * N * sizeof(float);
    Q6K_DISPATCH(dtype, q6k_launch(selective_scan_kernel<T>, grid, 128, smem, st, (const T*)u, dt_raw, dt_bias, proj, ldp, b_col, c_col, A,
                                   Dskip, xz, ldx, z_col, state, tail, q_start, slot_ids, (T*)out, C, N, L, taps););
    return q6k_check_launch("selective_scan");
}

// out[t, j] = dtype(src[t, col0 + j]), j < n: a few columns of an FP32 product as the next product's operand.
Q6K_API int q6k_cast_columns(const float* src, int ld, int col0, int n, void* out, int rows, int dtype, cudaStream_t st) {
    if (rows == 0 || n == 0) return 0;
    Q6K_REQUIRE(rows > 0 && n > 0 && col0 >= 0 && col0 + n <= ld, "cast_columns: columns %d..%d of %d", col0, col0 + n, ld);
    const size_t total = (size_t)rows * n;
    Q6K_DISPATCH(dtype, q6k_launch(cast_columns_kernel<T>, dim3((unsigned)((total + 255) / 256)), 256, 0, st, src, ld, col0, n, (T*)out, total););
    return q6k_check_launch("cast_columns");
}
