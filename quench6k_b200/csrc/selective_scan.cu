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
//
// A long portion is walked in segments of `seg_len` tokens by different blocks (the recurrence is linear in S, so a
// segment's effect on the state is a pair: the state it builds from zero and the sum of dt A over it, whose exponential
// is the decay it applies to what came before).  A first launch (MODE 1) leaves that pair per segment; the second (MODE 2)
// folds the pairs of the segments before its own into the state it starts from, in order, and then runs as the single
// launch (MODE 0) does.  This only regroups the sums of the recurrence: the result differs by rounding.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;
constexpr int SCAN_TILE = 32;      // tokens whose inputs are staged in shared memory at a time
constexpr int MAX_PER_LANE = 8;    // states per lane

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
// exp(x) - 1 for x <= 0 with a relative error near 1e-7: down to -1/4 the Taylor series in x (its truncation is below
// x^7 / 40320), beyond that expf(x) - 1, where the exponential's rounding is small beside its distance from 1.
// FAST (bfloat16 operands, whose own rounding is four orders of magnitude above it): the hardware exponential beyond -1/4
// (a few units in the last place of the exponential) and two terms fewer in the series.
template <bool FAST>
__device__ __forceinline__ float decay_minus_one(float x) {
    float p = FAST ? fmaf(x, 1.0f / 120.0f, 1.0f / 24.0f) : fmaf(x, fmaf(x, fmaf(x, 1.0f / 5040.0f, 1.0f / 720.0f), 1.0f / 120.0f), 1.0f / 24.0f);
    p = fmaf(x, p, 1.0f / 6.0f);
    p = fmaf(x, p, 0.5f);
    p = fmaf(x, p, 1.0f);
    return x > -0.25f ? x * p : (FAST ? __expf(x) : expf(x)) - 1.0f;
}

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

// grid (R, ceil(C / (128 / L)), segments), 128 threads; dynamic shared memory SCAN_TILE * (2 N + 4 * 128 / L) floats.
// ws (MODE 1, 2): per segment slot q = seg_base[r] + segment, [q][2][C][N] (the state built from zero, the sum of dt A),
// then per request [r][C][N], the state the step found in the request's slot.
template <typename T, int MODE>
__global__ void __launch_bounds__(128) selective_scan_kernel(const T* u, const float* dt_raw, const float* dt_bias, const float* proj, int ldp,
                                                             int b_col, int c_col, const float* A, const float* Dskip, const float* xz,
                                                             int ldx, int z_col, float* state, float* tail, const int* q_start,
                                                             const int* slot_ids, T* out, int C, int N, int L, int taps, float* ws,
                                                             const int* seg_base, int seg_len, int seg_slots) {
    pdl_enter();
    extern __shared__ float bc[];              // [SCAN_TILE][N] of B, the same of C, then four [SCAN_TILE][channels of the block]
    const int r = blockIdx.x, seg = MODE == 0 ? 0 : blockIdx.z;
    const int per_block = blockDim.x / L;
    const int c = blockIdx.y * per_block + threadIdx.x / L, sub = threadIdx.x % L;
    const bool live = c < C;
    const int first_req = q_start[r], n_req = q_start[r + 1] - first_req, slot = slot_ids[r];
    const int t_begin = MODE == 0 ? 0 : seg * seg_len;
    if (MODE != 0 && t_begin >= n_req) return;
    const int n_tok = MODE == 0 ? n_req : min(n_req - t_begin, seg_len);       // this block's tokens
    const int first = first_req + t_begin;
    const bool last_segment = t_begin + n_tok == n_req;
    const size_t CN = (size_t)C * N, own = ((size_t)(live ? c : 0)) * N;
    float S[MAX_PER_LANE], a[MAX_PER_LANE], dsum[MAX_PER_LANE];
    float* Sg = state + (size_t)slot * CN + own;
    float* seg_pair = MODE == 0 ? nullptr : ws + (size_t)(seg_base[r] + seg) * 2 * CN + own;
    float* found = MODE == 0 ? nullptr : ws + (size_t)seg_slots * 2 * CN + (size_t)r * CN + own;
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
        const int n = sub + L * k;
        const bool has = live && n < N;
        a[k] = has ? A[(size_t)c * N + n] : 0.0f;
        dsum[k] = 0.0f;
        if (MODE == 0) {
            S[k] = has ? Sg[n] : 0.0f;
        } else if (MODE == 1) {
            S[k] = 0.0f;
            if (has && seg == 0) found[n] = Sg[n];
        } else {
            S[k] = has ? found[n] : 0.0f;
            const float* pair = ws + (size_t)seg_base[r] * 2 * CN + own;
            for (int q = 0; q < seg; ++q, pair += 2 * CN)
                if (has) S[k] = fmaf(expm1f(pair[CN + n]), S[k], S[k]) + pair[n];
        }
    }
    if (MODE == 1 && last_segment) return;     // no later segment folds this one (segment 0 has left the state it found)
    // Per tile of SCAN_TILE tokens the block first makes, once per (token, channel) and with coalesced loads, what the
    // recurrence needs of them: dt = softplus(dt_raw + bias), dt u, the gate silu(z) and the skip D u; then B and C.
    float* s_dt = bc + 2 * SCAN_TILE * N;          // [SCAN_TILE][per_block]
    float* s_du = s_dt + SCAN_TILE * per_block;
    float* s_gate = s_du + SCAN_TILE * per_block;
    float* s_skip = s_gate + SCAN_TILE * per_block;
    const int c0 = blockIdx.y * per_block, cc = threadIdx.x / L;
    for (int t0 = 0; t0 < n_tok; t0 += SCAN_TILE) {
        const int nt = min(SCAN_TILE, n_tok - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
            const int tt = i / N, n = i % N;
            const float* pr = proj + (size_t)(first + t0 + tt) * ldp;
            bc[i] = pr[b_col + n];
            bc[SCAN_TILE * N + i] = pr[c_col + n];
        }
        for (int i = threadIdx.x; i < nt * per_block; i += blockDim.x) {
            const int tt = i / per_block, ch = c0 + i % per_block;
            if (ch < C) {
                const size_t row = (size_t)(first + t0 + tt);
                const float dt = softplus_f(dt_raw[row * C + ch] + dt_bias[ch]);
                const float uu = to_f32(u[row * C + ch]);
                s_dt[i] = dt;
                s_du[i] = dt * uu;
                if (MODE != 1) {
                    s_gate[i] = silu_f(xz[row * ldx + z_col + ch]);
                    s_skip[i] = Dskip[ch] * uu;
                }
            }
        }
        __syncthreads();
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt) {
            const float dt = s_dt[tt * per_block + cc], du = s_du[tt * per_block + cc];
            const float* Bt = bc + tt * N;
            const float* Ct = bc + SCAN_TILE * N + tt * N;
            float y = 0.0f;
#pragma unroll
            for (int k = 0; k < MAX_PER_LANE; ++k) {
                const int n = sub + L * k;
                if (n < N) {
                    // exp(dt A) S as S + expm1(dt A) S: a decay close to 1 keeps its distance from 1 to full precision, so
                    // that no rounding of the factor itself (always the same way for a given dt A) adds up over a long context
                    const float da = dt * a[k];
                    S[k] = fmaf(decay_minus_one<sizeof(T) == 2>(da), S[k], S[k]) + du * Bt[n];
                    if (MODE == 1) dsum[k] += da;
                    else y = fmaf(S[k], Ct[n], y);
                }
            }
            if (MODE != 1) {
                for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (live && sub == 0)
                    out[(size_t)(first + t0 + tt) * C + c] = from_f32<T>((y + s_skip[tt * per_block + cc]) * s_gate[tt * per_block + cc]);
            }
        }
    }
    if (!live) return;
    if (MODE == 1) {
#pragma unroll
        for (int k = 0; k < MAX_PER_LANE; ++k) {
            const int n = sub + L * k;
            if (n < N) {
                seg_pair[n] = S[k];
                seg_pair[CN + n] = dsum[k];
            }
        }
        return;
    }
    if (!last_segment) return;
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
                const int src = n_req - (taps - 1) + j;          // index within the portion
                keep[j] = src >= 0 ? xz[(size_t)(first_req + src) * ldx + c] : tl[(size_t)(j + n_req) * C];
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

// How many lanes share a channel for N states: the least power of two that leaves each lane at most eight (independent
// chains of the recurrence in one thread hide each other's latency; segments and channels supply the threads).
Q6K_API int q6k_selective_scan_lanes(int N) {
    int L = 1;
    while (L < 32 && L * MAX_PER_LANE < N) L *= 2;
    return L;
}

// u: dtype [T, C] (the convolution's result); dt_raw: FP32 [T, C]; proj: FP32 [T, ldp] with B in columns b_col.. and C in
// c_col.. (N each); A: FP32 [C, N] (negative); Dskip: FP32 [C]; xz: FP32 [T, ldx] with the convolution's inputs in columns
// 0.. and the gate z in columns z_col..; state: FP32 [slots, C, N]; tail: FP32 [slots, taps-1, C]; out: dtype [T, C].
// Tokens per segment when a portion is walked by several blocks.
Q6K_API int q6k_selective_scan_segment() { return 64; }

// Floats of scratch for `seg_slots` segments in all and R requests.
Q6K_API long long q6k_selective_scan_workspace(int seg_slots, int R, int C, int N) { return ((long long)seg_slots * 2 + R) * C * N; }

// segments > 1: portions are walked in segments of q6k_selective_scan_segment() tokens (`segments`: the most of any request;
// seg_base: int32 [R], the first segment slot of each request; seg_slots: their total; ws: the scratch above).
Q6K_API int q6k_selective_scan(const void* u, const float* dt_raw, const float* dt_bias, const float* proj, int ldp, int b_col, int c_col,
                               const float* A, const float* Dskip, const float* xz, int ldx, int z_col, float* state, float* tail,
                               const int* q_start, const int* slot_ids, void* out, int R, int C, int N, int taps, int dtype,
                               int segments, const int* seg_base, int seg_slots, float* ws, cudaStream_t st) {
    if (R == 0) return 0;
    const int L = q6k_selective_scan_lanes(N);
    Q6K_REQUIRE(R > 0 && C > 0 && N > 0 && N <= L * MAX_PER_LANE, "selective_scan: bad sizes R=%d C=%d N=%d (at most %d states)", R, C, N,
                32 * MAX_PER_LANE);
    Q6K_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "selective_scan: %d taps (at most %d)", taps, MAX_TAPS);
    const int per_block = 128 / L;
    dim3 grid(R, (C + per_block - 1) / per_block);
    Q6K_REQUIRE(grid.y <= 65535, "selective_scan: %d channels exceed the grid limit", C);
    const size_t smem = (size_t)SCAN_TILE * (2 * N + 4 * per_block) * sizeof(float);
    const int seg_len = q6k_selective_scan_segment();
#define SCAN_LAUNCH(MODE, GRID)                                                                                                      \
    Q6K_DISPATCH(dtype, if (smem > 48 * 1024) cudaFuncSetAttribute(selective_scan_kernel<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                 q6k_launch(selective_scan_kernel<T, MODE>, GRID, 128, smem, st, (const T*)u, dt_raw, dt_bias, proj, ldp, b_col, c_col, A, \
                                   Dskip, xz, ldx, z_col, state, tail, q_start, slot_ids, (T*)out, C, N, L, taps, ws, seg_base, seg_len, seg_slots););
    if (segments <= 1) {
        SCAN_LAUNCH(0, grid);
        return q6k_check_launch("selective_scan");
    }
    Q6K_REQUIRE(seg_base && ws && seg_slots > 0 && segments <= 65535, "selective_scan: segments need their slots and scratch");
    dim3 grid3(R, grid.y, segments);
    SCAN_LAUNCH(1, grid3);
    if (int rc = q6k_check_launch("selective_scan (segments)")) return rc;
    SCAN_LAUNCH(2, grid3);
#undef SCAN_LAUNCH
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
