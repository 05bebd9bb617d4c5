// Attention over the paged cache with a modified score: keys and values in planes of their own
// (their widths may differ), and between the dot product and the softmax any of
//   a cap          s <- cap * tanh(s / cap),
//   a distance bias s <- s - slope[head] * (pos_query - pos_key),
//   a chunk mask   keys only from the query's own chunk of `chunk` positions (counted from 0),
//   a window       keys pos - window + 1 .. pos,
//   a sink         one more term exp(0) in the softmax's denominator that carries no value,
// and after the softmax an output gate: out *= sigmoid(gate).  Every constant is an argument; a
// zero (or a null pointer) switches its step off, and with all of them off this is plain causal
// attention.
//
// Three kernels.  `qkv_unit_store`: per-head RMS norm of queries and keys (with or without gains)
// and the write of keys and values into their pages.  `attention_biased_general`: one block per
// (token, query head), any widths up to 512, float32 or bfloat16; the float32 path and the fallback.
// `attention_biased_prefill`: bfloat16 prompt portions on mma.sync tiles, 64 query rows of one head
// per block, widths up to 128 (padded with zeros to 64 or 128 in shared memory).
// `attention_biased_decode`: one-token rows, one block per (row, key/value head): the keys and values
// are read once for all query heads of the group, 16 bytes per lane.
//
// Scores, the cap, the bias, the softmax and the gate are float32 in both storage types.  The order of
// the additions for a (request, position, head) depends on the position and the constants only.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace tllm {

struct ScoreMod {
    float scale, softcap;
    int chunk, window, sink;
};

__device__ __forceinline__ int first_key(int pos, const ScoreMod& m) {
    int lo = 0;
    if (m.chunk > 0) lo = (pos / m.chunk) * m.chunk;
    if (m.window > 0 && pos - m.window + 1 > lo) lo = pos - m.window + 1;
    return lo;
}

__device__ __forceinline__ float mod_score(float dot, float slope, int dist, const ScoreMod& m) {
    float s = dot * m.scale;
    if (m.softcap > 0.0f) s = m.softcap * tanhf(s / m.softcap);
    return s - slope * (float)dist;
}

// ---------------------------------------------------------------- norm of q and k, write of k and v
// proj[t] = q heads | k heads | v heads | (anything else).  One warp per head of a token.
template <typename T>
__global__ void qkv_unit_store_kernel(const T* proj, int row_stride, const T* __restrict__ q_gain,
                                      const T* __restrict__ k_gain, float eps, int do_norm,
                                      const int* __restrict__ positions, const int* __restrict__ token_slot,
                                      const int* __restrict__ block_table, int max_pages, int page_size,
                                      T* k_plane, T* v_plane, long long page_stride, T* q_out,
                                      int q_heads, int kv_heads, int dk, int dv, int store) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int pos = positions[t];
    const T* row = proj + (size_t)t * row_stride;
    long long page_base = -1;
    int in_page = 0;
    if (store) {
        const int page = block_table[(size_t)slot * max_pages + pos / page_size];
        page_base = (long long)page * page_stride;
        in_page = pos % page_size;
        if (page < 0) store = 0;          // no page held: nothing to write (the host reserves before a step)
    }
    const int total = q_heads + 2 * kv_heads;
    for (int head = warp; head < total; head += warps) {
        if (head < q_heads + kv_heads) {
            const bool is_q = head < q_heads;
            const T* src = row + (size_t)head * dk;
            const T* gain = is_q ? q_gain : k_gain;
            float sum = 0.0f;
            for (int e = lane; e < dk; e += 32) {
                const float x = to_f32<T>(src[e]);
                sum += x * x;
            }
            sum = warp_sum(sum);
            const float sc = do_norm ? 1.0f / sqrtf(sum / (float)dk + eps) : 1.0f;
            T* dst;
            if (is_q) dst = q_out + ((size_t)t * q_heads + head) * dk;
            else if (store) dst = k_plane + page_base + ((size_t)(head - q_heads) * page_size + in_page) * dk;
            else continue;
            for (int e = lane; e < dk; e += 32) {
                float x = to_f32<T>(src[e]) * sc;
                if (gain != nullptr && do_norm) x *= to_f32<T>(gain[e]);
                dst[e] = from_f32<T>(x);
            }
        } else if (store) {
            const int g = head - q_heads - kv_heads;
            const T* src = row + (size_t)(q_heads + kv_heads) * dk + (size_t)g * dv;
            T* dst = v_plane + page_base + ((size_t)g * page_size + in_page) * dv;
            for (int e = lane; e < dv; e += 32) dst[e] = src[e];
        }
    }
}

// ---------------------------------------------------------------- general kernel
constexpr int kGenWarps = 4;

template <typename T, int CK, int CV>
__global__ void attention_biased_general_kernel(
    const T* q, const T* k_plane, const T* v_plane, long long page_stride,
    const int* __restrict__ positions, const int* __restrict__ token_slot,
    const int* __restrict__ block_table, int max_pages, int page_size, int q_heads, int kv_heads,
    int dk, int dv, ScoreMod mod, const float* __restrict__ slopes, const T* gate, int gate_stride,
    T* __restrict__ out) {
    extern __shared__ float smem[];
    TLLM_PDL_ENTER();
    float* qs = smem;                             // [dk]
    float* acc_s = smem + dk;                     // [warps][dv]
    float* m_s = acc_s + kGenWarps * dv;          // [warps]
    float* l_s = m_s + kGenWarps;                 // [warps]

    const int head = blockIdx.x, t = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* dst = out + ((size_t)t * q_heads + head) * dv;
    const int slot = token_slot[t];
    if (slot < 0) {
        for (int e = threadIdx.x; e < dv; e += blockDim.x) dst[e] = from_f32<T>(0.0f);
        return;
    }
    const int pos = positions[t];
    const int lo = first_key(pos, mod);
    const int g = head / (q_heads / kv_heads);
    const float slope = slopes != nullptr ? slopes[head] : 0.0f;
    const T* qsrc = q + ((size_t)t * q_heads + head) * dk;
    for (int e = threadIdx.x; e < dk; e += blockDim.x) qs[e] = to_f32<T>(qsrc[e]);
    __syncthreads();

    const int* table = block_table + (size_t)slot * max_pages;
    // the sink is a key of score 0 without a value; warp 0 starts from it
    float m = (mod.sink && warp == 0) ? 0.0f : -INFINITY;
    float l = (mod.sink && warp == 0) ? 1.0f : 0.0f;
    float acc[CV];
#pragma unroll
    for (int c = 0; c < CV; ++c) acc[c] = 0.0f;

    for (int j = lo + warp; j <= pos; j += kGenWarps) {
        const int page = table[j / page_size];
        if (page < 0) continue;
        const size_t in_page = (size_t)g * page_size + (j % page_size);
        const T* kp = k_plane + (long long)page * page_stride + in_page * dk;
        const T* vp = v_plane + (long long)page * page_stride + in_page * dv;
        float dot = 0.0f;
#pragma unroll
        for (int c = 0; c < CK; ++c) {
            const int e = lane + 32 * c;
            if (e < dk) dot += qs[e] * to_f32<T>(kp[e]);
        }
        dot = warp_sum(dot);
        const float s = mod_score(dot, slope, pos - j, mod);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int c = 0; c < CV; ++c) {
            const int e = lane + 32 * c;
            if (e < dv) acc[c] = acc[c] * corr + p * to_f32<T>(vp[e]);
        }
        m = m_new;
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int c = 0; c < CV; ++c) {
        const int e = lane + 32 * c;
        if (e < dv) acc_s[warp * dv + e] = acc[c];
    }
    __syncthreads();
    float mm = m_s[0];
#pragma unroll
    for (int w = 1; w < kGenWarps; ++w) mm = fmaxf(mm, m_s[w]);
    float w_scale[kGenWarps], total = 0.0f;
#pragma unroll
    for (int w = 0; w < kGenWarps; ++w) {
        w_scale[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - mm);
        total += l_s[w] * w_scale[w];
    }
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    const T* grow = gate != nullptr ? gate + (size_t)t * gate_stride + (size_t)head * dv : nullptr;
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kGenWarps; ++w) v += acc_s[w * dv + e] * w_scale[w];
        v *= inv;
        if (grow != nullptr) v *= 1.0f / (1.0f + expf(-to_f32<T>(grow[e])));
        dst[e] = from_f32<T>(v);
    }
}

template <typename T>
static int launch_general(const void* q, const void* kp, const void* vp, long long page_stride,
                          const int* positions, const int* token_slot, const int* block_table,
                          int max_pages, int page_size, int tokens, int q_heads, int kv_heads, int dk,
                          int dv, ScoreMod mod, const float* slopes, const void* gate, int gate_stride,
                          void* out, cudaStream_t stream) {
    const dim3 grid(q_heads, tokens), block(kGenWarps * 32);
    const size_t smem = ((size_t)dk + (size_t)kGenWarps * dv + 2 * kGenWarps) * sizeof(float);
    const int ck = (dk + 31) / 32, cv = (dv + 31) / 32;
    const int c = ck > cv ? ck : cv;
#define LAUNCH(C)                                                                                           \
    launch_pdl(kPdlAttention, attention_biased_general_kernel<T, C, C>, grid, block, smem, stream,          \
               (const T*)q, (const T*)kp, (const T*)vp, page_stride, positions, token_slot, block_table,    \
               max_pages, page_size, q_heads, kv_heads, dk, dv, mod, slopes, (const T*)gate, gate_stride, (T*)out)
    if (c <= 1) LAUNCH(1);
    else if (c <= 2) LAUNCH(2);
    else if (c <= 4) LAUNCH(4);
    else if (c <= 8) LAUNCH(8);
    else LAUNCH(16);
#undef LAUNCH
    return finish_launch("attention_biased_general");
}

}  // namespace tllm

using namespace tllm;

extern "C" {

int tllm_qkv_unit_store(const void* proj, int row_stride, const void* q_gain, const void* k_gain, float eps,
                        int do_norm, const int* positions, const int* token_slot, const int* block_table,
                        int max_pages, int page_size, void* k_plane, void* v_plane, long long page_stride,
                        void* q_out, int dtype, int tokens, int q_heads, int kv_heads, int dk, int dv,
                        int store, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && dk > 0 && dv > 0, "qkv_unit_store: bad sizes");
    TLLM_REQUIRE(row_stride >= (q_heads + kv_heads) * dk + kv_heads * dv, "qkv_unit_store: rows of %d are too short", row_stride);
    TLLM_REQUIRE(!do_norm || eps > 0.0f, "qkv_unit_store: eps must be positive");
    TLLM_REQUIRE(!store || (k_plane && v_plane && block_table && page_size > 0 && max_pages > 0),
                 "qkv_unit_store: no cache to write to");
    TLLM_REQUIRE(q_out != nullptr, "qkv_unit_store: no place for the queries");
    if (tokens == 0) return 0;
    const int heads = q_heads + 2 * kv_heads;
    const int warps = heads >= 8 ? 8 : (heads >= 4 ? 4 : 2);
#define STORE(T)                                                                                              \
    launch_pdl(kPdlQk, qkv_unit_store_kernel<T>, dim3(tokens), dim3(warps * 32), 0, stream, (const T*)proj,   \
               row_stride, (const T*)q_gain, (const T*)k_gain, eps, do_norm, positions, token_slot,           \
               block_table, max_pages, page_size, (T*)k_plane, (T*)v_plane, page_stride, (T*)q_out, q_heads,  \
               kv_heads, dk, dv, store)
    if (dtype == kBF16) STORE(bf16);
    else if (dtype == kF32) STORE(float);
    else TLLM_REQUIRE(false, "qkv_unit_store: unknown dtype %d", dtype);
#undef STORE
    return finish_launch("qkv_unit_store");
}

int tllm_attention_biased_general(
    const void* q, const void* k_plane, const void* v_plane, long long page_stride, const int* positions,
    const int* token_slot, const int* block_table, int max_pages, int page_size, int dtype, int tokens,
    int q_heads, int kv_heads, int dk, int dv, float scale, float softcap, int chunk, int window, int sink,
    const float* slopes, const void* gate, int gate_stride, void* out, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
                 "attention_biased: %d query heads over %d key/value heads", q_heads, kv_heads);
    TLLM_REQUIRE(dk > 0 && dk <= 512 && dv > 0 && dv <= 512, "attention_biased: widths %d, %d outside 1..512", dk, dv);
    TLLM_REQUIRE(page_size > 0 && max_pages > 0, "attention_biased: bad page geometry");
    TLLM_REQUIRE(tokens <= 65535, "attention_biased: %d tokens in one step exceed 65535", tokens);
    TLLM_REQUIRE(chunk >= 0 && window >= 0 && softcap >= 0.0f, "attention_biased: negative constant");
    if (tokens == 0) return 0;
    const ScoreMod mod{scale, softcap, chunk, window, sink ? 1 : 0};
    if (dtype == kBF16)
        return launch_general<bf16>(q, k_plane, v_plane, page_stride, positions, token_slot, block_table, max_pages,
                                    page_size, tokens, q_heads, kv_heads, dk, dv, mod, slopes, gate, gate_stride, out, stream);
    if (dtype == kF32)
        return launch_general<float>(q, k_plane, v_plane, page_stride, positions, token_slot, block_table, max_pages,
                                     page_size, tokens, q_heads, kv_heads, dk, dv, mod, slopes, gate, gate_stride, out, stream);
    TLLM_REQUIRE(false, "attention_biased: unknown dtype %d", dtype);
}

}  // extern "C"
