// The delta rule with a decay per head and key channel, as a recurrence over a state S [dk, dv] per
// (request, head) that lives in float32 and is carried from step to step:
//
//   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t.
//
// Three kernels serve a step, prompt portions and single tokens alike:
//
//   delta_prepare  one block per token: the short causal convolution of the q, k and v channels (taps
//                  reaching before the portion come from the request's state), SiLU, unit length of q
//                  and k per head (q times a scale), g = exp(-rate_h softplus(a + bias)) and
//                  beta = sigmoid(b); all results in float32.
//   delta_scan     one block per (portion, head, group of value columns): a column of S is independent of
//                  the others, so a thread keeps a slice of one column in registers (the dk rows are dealt
//                  to R neighbouring lanes, which add their partial dot products with shuffles) and walks
//                  the portion's tokens, which are staged in shared memory sixteen at a time.
//   delta_finish   one block per token: o divided by its root mean square per head, times a weight, times
//                  sigmoid(gate); the block of a portion's last token also moves the convolution's
//                  window of the request's state on.
//
// State of a request: [heads][per][dv][R] floats of S (row i = il * R + r; rows past dk stay zero), then
// [taps - 1][channels] inputs of the convolution, the newest last.  R and per follow from dk alone
// (`tllm_delta_rule_lanes`), so every step of a request finds the layout the last one left.
#include "common.cuh"

namespace tllm {

constexpr int kScanMaxPer = 16;     // rows of a column that one thread keeps
constexpr int kScanChunk = 16;      // tokens staged at a time

static inline int delta_lanes(int dk) {
    int r = 4;
    while (r < 32 && (dk + r - 1) / r > kScanMaxPer) r *= 2;
    return r;
}

__device__ __forceinline__ float softplus_f32(float x) {
    return x > 20.0f ? x : log1pf(expf(x));
}

// ---------------------------------------------------------------- prepare
template <typename T>
__global__ void delta_prepare_kernel(const T* proj, int ld, const T* __restrict__ conv_w, int taps,
                                     const float* a, int lda, const float* __restrict__ dt_bias,
                                     const float* __restrict__ rate, const int* __restrict__ token_slot,
                                     const float* state, long long state_stride, long long tail_off,
                                     int heads, int kv_heads, int dk, int dv, float q_scale, float unit_eps,
                                     float* qn, float* kn, float* vv, float* decay, float* beta, int n_rows) {
    extern __shared__ float y[];                 // [channels] after convolution and SiLU
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int qk = kv_heads * dk, channels = 2 * qk + heads * dv;
    int back = 0;                                // rows before this one that belong to the same portion
    for (int j = 1; j < taps; ++j) {
        if (t - j >= 0 && token_slot[t - j] == slot) back = j;
        else break;
    }
    const float* tail = state + (long long)slot * state_stride + tail_off;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const float w = to_f32<T>(conv_w[(size_t)c * taps + (taps - 1 - j)]);
            float x;
            if (j <= back) x = to_f32<T>(proj[(size_t)(t - j) * ld + c]);
            else x = tail[(size_t)(taps - 1 - (j - back)) * channels + c];
            acc += w * x;
        }
        y[c] = acc / (1.0f + expf(-acc));
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int u = warp; u < 2 * kv_heads; u += warps) {          // q heads, then k heads
        const float* src = y + (size_t)u * dk;
        float sum = 0.0f;
        for (int e = lane; e < dk; e += 32) sum += src[e] * src[e];
        sum = warp_sum(sum);
        const bool is_q = u < kv_heads;
        const float sc = (is_q ? q_scale : 1.0f) / sqrtf(sum + unit_eps);
        float* dst = is_q ? qn + (size_t)t * qk + (size_t)u * dk : kn + (size_t)t * qk + (size_t)(u - kv_heads) * dk;
        for (int e = lane; e < dk; e += 32) dst[e] = src[e] * sc;
    }
    for (int e = threadIdx.x; e < heads * dv; e += blockDim.x) vv[(size_t)t * heads * dv + e] = y[2 * qk + e];
    for (int e = threadIdx.x; e < heads * dk; e += blockDim.x) {
        const float x = a[(size_t)t * lda + e] + dt_bias[e];
        decay[(size_t)t * heads * dk + e] = expf(-rate[e / dk] * softplus_f32(x));
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float b = to_f32<T>(proj[(size_t)t * ld + channels + h]);
        beta[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-b));
    }
}

// ---------------------------------------------------------------- scan
template <int R>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = R / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int R>
__global__ void delta_scan_kernel(const int* __restrict__ seg_info, const int* __restrict__ token_slot,
                                  const float* qn, const float* kn, const float* vv, const float* decay,
                                  const float* beta, float* state, long long state_stride, int heads,
                                  int kv_heads, int dk, int dv, int cols, float* o_raw) {
    extern __shared__ float sm[];
    TLLM_PDL_ENTER();
    const int seg = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
    int slot, start, len;
    if (seg_info != nullptr) {
        slot = seg_info[4 * seg]; start = seg_info[4 * seg + 1]; len = seg_info[4 * seg + 2];
    } else {
        slot = token_slot[seg]; start = seg; len = 1;
    }
    if (slot < 0 || len <= 0) return;
    const int per = (dk + R - 1) / R, dkp = per * R;
    const int r = threadIdx.x % R, jl = threadIdx.x / R;       // lane of the column, column of the block
    const int j = col0 + jl;
    const bool live = jl < cols && j < dv;
    const int kvh = head / (heads / kv_heads);
    float* k_s = sm;                                  // [chunk][dkp]
    float* q_s = k_s + kScanChunk * dkp;              // [chunk][dkp]
    float* g_s = q_s + kScanChunk * dkp;              // [chunk][dkp]
    float* v_s = g_s + kScanChunk * dkp;              // [chunk][cols]
    float* o_s = v_s + kScanChunk * cols;             // [chunk][cols]
    float* b_s = o_s + kScanChunk * cols;             // [chunk]

    float* st = state + (long long)slot * state_stride + (size_t)head * per * dv * R;
    float S[kScanMaxPer];
#pragma unroll
    for (int il = 0; il < kScanMaxPer; ++il)
        S[il] = (live && il < per) ? st[((size_t)il * dv + j) * R + r] : 0.0f;

    for (int c0 = 0; c0 < len; c0 += kScanChunk) {
        const int n = min(kScanChunk, len - c0);
        __syncthreads();                              // the chunk before has been written out
        for (int i = threadIdx.x; i < n * dkp; i += blockDim.x) {
            const int tt = i / dkp, e = i - tt * dkp;
            const size_t row = (size_t)(start + c0 + tt);
            const bool in = e < dk;
            k_s[i] = in ? kn[(row * kv_heads + kvh) * dk + e] : 0.0f;
            q_s[i] = in ? qn[(row * kv_heads + kvh) * dk + e] : 0.0f;
            g_s[i] = in ? decay[(row * heads + head) * dk + e] : 0.0f;
        }
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, e = i - tt * cols;
            v_s[i] = (col0 + e < dv) ? vv[((size_t)(start + c0 + tt) * heads + head) * dv + col0 + e] : 0.0f;
        }
        for (int i = threadIdx.x; i < n; i += blockDim.x) b_s[i] = beta[(size_t)(start + c0 + i) * heads + head];
        __syncthreads();
        {   // every thread walks the tokens (the shuffles want whole warps); one without a column carries zeros
            for (int tt = 0; tt < n; ++tt) {
                const float* kr = k_s + tt * dkp + r;
                const float* qr = q_s + tt * dkp + r;
                const float* gr = g_s + tt * dkp + r;
                float kk[kScanMaxPer];
                float dot = 0.0f;
#pragma unroll
                for (int il = 0; il < kScanMaxPer; ++il)
                    if (il < per) {
                        kk[il] = kr[il * R];
                        S[il] *= gr[il * R];
                        dot += S[il] * kk[il];
                    }
                dot = lanes_sum<R>(dot);
                const float u = b_s[tt] * (v_s[tt * cols + jl] - dot);
                float oq = 0.0f;
#pragma unroll
                for (int il = 0; il < kScanMaxPer; ++il)
                    if (il < per) {
                        S[il] += kk[il] * u;
                        oq += S[il] * qr[il * R];
                    }
                oq = lanes_sum<R>(oq);
                if (r == 0 && live) o_s[tt * cols + jl] = oq;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, e = i - tt * cols;
            if (col0 + e < dv) o_raw[((size_t)(start + c0 + tt) * heads + head) * dv + col0 + e] = o_s[i];
        }
    }
    if (live) {
#pragma unroll
        for (int il = 0; il < kScanMaxPer; ++il)
            if (il < per) st[((size_t)il * dv + j) * R + r] = S[il];
    }
}

// ---------------------------------------------------------------- finish
template <typename T>
__global__ void delta_finish_kernel(const float* o_raw, const float* gate, int ldg, const float* __restrict__ weight,
                                    float eps, const int* __restrict__ token_slot, int n_rows, int heads, int dv,
                                    T* out, const T* proj, int ld, int channels, int taps, float* state,
                                    long long state_stride, long long tail_off) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    if (slot < 0) {
        for (int e = threadIdx.x; e < heads * dv; e += blockDim.x) out[(size_t)t * heads * dv + e] = from_f32<T>(0.0f);
        return;
    }
    for (int h = warp; h < heads; h += warps) {
        const float* src = o_raw + ((size_t)t * heads + h) * dv;
        float sum = 0.0f;
        for (int e = lane; e < dv; e += 32) sum += src[e] * src[e];
        sum = warp_sum(sum);
        const float sc = 1.0f / sqrtf(sum / (float)dv + eps);
        for (int e = lane; e < dv; e += 32) {
            const float g = gate[(size_t)t * ldg + (size_t)h * dv + e];
            out[((size_t)t * heads + h) * dv + e] = from_f32<T>(src[e] * sc * weight[e] / (1.0f + expf(-g)));
        }
    }
    // the portion's last row moves the convolution's window on: its taps - 1 newest inputs
    if (taps > 1 && (t + 1 >= n_rows || token_slot[t + 1] != slot)) {
        int len = 1;                                 // rows of the portion, as far as the window reaches
        while (len < taps - 1 && t - len >= 0 && token_slot[t - len] == slot) ++len;
        float* tail = state + (long long)slot * state_stride + tail_off;
        const int keep = taps - 1;
        for (int c = threadIdx.x; c < channels; c += blockDim.x) {
            for (int i = 0; i < keep; ++i) {         // ascending: an old entry is read before its place is written
                const int from_end = keep - i;       // this entry is the from_end-th newest input
                float x;
                if (from_end <= len) x = to_f32<T>(proj[(size_t)(t + 1 - from_end) * ld + c]);
                else x = tail[(size_t)(i + len) * channels + c];
                tail[(size_t)i * channels + c] = x;
            }
        }
    }
}

}  // namespace tllm

using namespace tllm;

extern "C" {

// Lanes that share a column of the state for keys of width dk (the state's layout depends on it).
int tllm_delta_rule_lanes(int dk) { return delta_lanes(dk); }

// Floats of one request's state: S of every head in the scan's layout, then the convolution's window.
long long tllm_delta_rule_state_floats(int heads, int kv_heads, int dk, int dv, int taps) {
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    return (long long)heads * per * r * dv + (long long)(taps - 1) * (2 * kv_heads * dk + heads * dv);
}

int tllm_delta_prepare(const void* proj, int ld, int dtype, const void* conv_w, int taps, const float* a, int lda,
                       const float* dt_bias, const float* rate, const int* token_slot, const float* state,
                       long long state_stride, int heads, int kv_heads, int dk, int dv, float q_scale,
                       float unit_eps, float* qn, float* kn, float* vv, float* decay, float* beta, int n_rows,
                       cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0 && taps > 0,
                 "delta_prepare: bad sizes");
    const int channels = 2 * kv_heads * dk + heads * dv;
    TLLM_REQUIRE(ld >= channels + heads && lda >= heads * dk, "delta_prepare: rows too short");
    const size_t smem = (size_t)channels * sizeof(float);
    TLLM_REQUIRE(smem <= 200 * 1024, "delta_prepare: %d channels do not fit in shared memory", channels);
    if (n_rows == 0) return 0;
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    TLLM_REQUIRE(per <= kScanMaxPer, "delta_prepare: keys of width %d are too wide", dk);
    const long long tail_off = (long long)heads * per * r * dv;
#define PREP(T)                                                                                                  \
    do {                                                                                                         \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("delta_prepare: %s", cudaGetErrorString(e)); return (int)e; }      \
        }                                                                                                        \
        launch_pdl(kPdlOther, delta_prepare_kernel<T>, dim3(n_rows), dim3(256), smem, stream, (const T*)proj, ld, \
                   (const T*)conv_w, taps, a, lda, dt_bias, rate, token_slot, state, state_stride, tail_off,     \
                   heads, kv_heads, dk, dv, q_scale, unit_eps, qn, kn, vv, decay, beta, n_rows);                 \
    } while (0)
    if (dtype == kBF16) PREP(bf16);
    else if (dtype == kF32) PREP(float);
    else TLLM_REQUIRE(false, "delta_prepare: unknown dtype %d", dtype);
#undef PREP
    return finish_launch("delta_prepare");
}

// seg_info: int[segments][4] = slot, first row, length, first position; null: every row is a portion of one token.
int tllm_delta_scan(const int* seg_info, int segments, const int* token_slot, const float* qn, const float* kn,
                    const float* vv, const float* decay, const float* beta, float* state, long long state_stride,
                    int heads, int kv_heads, int dk, int dv, float* o_raw, cudaStream_t stream) {
    TLLM_REQUIRE(segments >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0,
                 "delta_scan: bad sizes");
    TLLM_REQUIRE(heads <= 65535, "delta_scan: %d heads", heads);
    if (segments == 0) return 0;
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    TLLM_REQUIRE(per <= kScanMaxPer, "delta_scan: keys of width %d are too wide", dk);
    // columns per block: whole warps, at most 256 threads, and at least two blocks per multiprocessor in all
    // where the value width allows it
    int cols = 256 / r;
    const int min_cols = 32 / r > 1 ? 32 / r : 1;
    const int sms = sm_count_cached() > 0 ? sm_count_cached() : 148;
    while (cols > min_cols && cols / 2 >= dv) cols /= 2;
    while (cols > min_cols && (long long)segments * heads * ((dv + cols - 1) / cols) < 2LL * sms) cols /= 2;
    const int col_blocks = (dv + cols - 1) / cols;
    const int threads = cols * r;
    const size_t smem = (size_t)kScanChunk * (3 * per * r + 2 * cols + 1) * sizeof(float);
    TLLM_REQUIRE(smem <= 200 * 1024 && col_blocks <= 65535, "delta_scan: sizes %d x %d do not fit", dk, dv);
#define SCAN(RR)                                                                                                 \
    do {                                                                                                         \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("delta_scan: %s", cudaGetErrorString(e)); return (int)e; }         \
        }                                                                                                        \
        launch_pdl(kPdlOther, delta_scan_kernel<RR>, dim3(segments, heads, col_blocks), dim3(threads), smem, stream, \
                   seg_info, token_slot, qn, kn, vv, decay, beta, state, state_stride, heads, kv_heads, dk, dv,  \
                   cols, o_raw);                                                                                 \
    } while (0)
    if (r == 4) SCAN(4);
    else if (r == 8) SCAN(8);
    else if (r == 16) SCAN(16);
    else SCAN(32);
#undef SCAN
    return finish_launch("delta_scan");
}

int tllm_delta_finish(const float* o_raw, const float* gate, int ldg, const float* weight, float eps,
                      const int* token_slot, int n_rows, int heads, int kv_heads, int dk, int dv, void* out,
                      int dtype, const void* proj, int ld, int taps, float* state, long long state_stride,
                      cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && heads > 0 && dv > 0 && eps > 0.0f && ldg >= heads * dv, "delta_finish: bad sizes");
    if (n_rows == 0) return 0;
    const int channels = 2 * kv_heads * dk + heads * dv;
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    const long long tail_off = (long long)heads * per * r * dv;
    if (dtype == kBF16)
        launch_pdl(kPdlOther, delta_finish_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, o_raw, gate, ldg, weight, eps,
                   token_slot, n_rows, heads, dv, (bf16*)out, (const bf16*)proj, ld, channels, taps, state, state_stride, tail_off);
    else if (dtype == kF32)
        launch_pdl(kPdlOther, delta_finish_kernel<float>, dim3(n_rows), dim3(256), 0, stream, o_raw, gate, ldg, weight, eps,
                   token_slot, n_rows, heads, dv, (float*)out, (const float*)proj, ld, channels, taps, state, state_stride, tail_off);
    else TLLM_REQUIRE(false, "delta_finish: unknown dtype %d", dtype);
    return finish_launch("delta_finish");
}

}  // extern "C"
