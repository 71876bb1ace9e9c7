// Plain paged attention: one block per (token, query head), any head size, any page
// size, float32 or bfloat16.  It is the 32-bit path's attention and the fallback for
// sizes the tensor-core kernels refuse.
//
// score = q·k * scale; query at position p sees keys max(0, p-window+1)..p of its own
// request (window 0 = all keys); softmax state and accumulators in 32-bit; the
// probability is rounded to the activation type before it multiplies V; the output is
// rounded once.  The value head size `dv` may differ from the query/key size `d`: a page holds
// the keys [kv head][slot][d] and then the values [kv head][slot][dv].
// Options: `softcap` c > 0 caps the scaled score, s <- c tanh(s / c); `sink` adds a key of score 0
// that has no value (one more term, exp(0), in the softmax's denominator); `gate` (with its row
// pitch) multiplies the output element by element with sigmoid(gate[t][h * dv + i]); `sink_logits`
// (one per query head) puts a learned logit in the place of the sink's 0, unscaled; `keep_first` n > 0
// (with a window) keeps keys 0..n-1 visible beside the window's.  Reference: src/sparseengine/kernels/triton/context_flashattention_nopad.py:92-127,
// src/sparseengine/kernels/triton/gqa_flash_decoding_stage1.py:69-120.
//
// A block-table entry outside [0, num_pages) is not followed: the key is left out and a code
// goes to the error word (the reference checks such indices on the host behind a debug
// switch, src/sparseengine/layers/attention_backend.py:155-215).
#include "common.cuh"

namespace se {

constexpr int kAttnWarps = 4;
constexpr int kMaxDimPerLane = 8;   // head_dim <= 256

template <typename T>
__global__ void paged_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                                             const int* __restrict__ table, int table_stride,
                                             const int* __restrict__ seq_rows, const int* __restrict__ token_seq,
                                             const int* __restrict__ positions, T* __restrict__ out, int hq, int hkv,
                                             int d, int dv, int page_size, float scale, int window, int num_pages,
                                             int* __restrict__ error, float softcap, int sink,
                                             const T* __restrict__ gate, int gate_pitch,
                                             const float* __restrict__ sink_logits, int keep_first) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = h / (hq / hkv);
    const int pos = positions[t];
    const int* row_table = table + (size_t)seq_rows[token_seq[t]] * table_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const size_t page_elems = (size_t)hkv * page_size * (d + dv);
    const size_t v_off = (size_t)hkv * page_size * d + (size_t)kvh * page_size * dv;
    const size_t head_off = (size_t)kvh * page_size * d;

    float qr[kMaxDimPerLane], acc[kMaxDimPerLane];
    const T* qp = q + ((size_t)t * hq + h) * d;
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) {
        const int dim = lane + 32 * i;
        qr[i] = dim < d ? to_float(qp[dim]) * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    // the keys in the order they are visited: the kept first ones that lie before the window, then the window's
    const int kept = min(keep_first, lo), seen = kept + pos - lo + 1;
    for (int n = warp; n < seen; n += kAttnWarps) {
        const int j = n < kept ? n : lo + n - kept;
        const int page = row_table[j / page_size];
        if (!page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_ATTN_PLAIN)) continue;     // warp-uniform: the key is left out
        const T* kp = cache + (size_t)page * page_elems + head_off + (size_t)(j % page_size) * d;
        const T* vp = cache + (size_t)page * page_elems + v_off + (size_t)(j % page_size) * dv;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxDimPerLane; ++i) {
            const int dim = lane + 32 * i;
            if (dim < d) s += qr[i] * to_float(kp[dim]);
        }
        s = warp_sum(s);
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);   // m = -inf on the first key: exp(-inf) = 0
        const float p = expf(s - m_new);
        const float pr = round_act<T>(p);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < kMaxDimPerLane; ++i) {
            const int dim = lane + 32 * i;
            if (dim < dv) acc[i] = acc[i] * corr + pr * to_float(vp[dim]);
        }
        m = m_new;
    }

    __shared__ float sm[kAttnWarps], sl[kAttnWarps];
    __shared__ float sacc[kAttnWarps][32 * kMaxDimPerLane];
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) sacc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mt = fmaxf(mt, sm[w]);
    const float sink_logit = sink_logits != nullptr ? sink_logits[h] : 0.f;
    if (sink) mt = fmaxf(mt, sink_logit);
    float lt = sink ? expf(sink_logit - mt) : 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) lt += sm[w] == -INFINITY ? 0.f : sl[w] * expf(sm[w] - mt);
    T* op = out + ((size_t)t * hq + h) * dv;
    for (int dim = threadIdx.x; dim < dv; dim += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) o += sm[w] == -INFINITY ? 0.f : sacc[w][dim] * expf(sm[w] - mt);
        o /= lt;
        if (gate != nullptr) o /= 1.f + expf(-to_float(gate[(size_t)t * gate_pitch + (size_t)h * dv + dim]));
        op[dim] = from_float<T>(o);
    }
}

}  // namespace se

extern "C" int se_paged_attention_plain(const void* q, const void* cache, const int* table, int table_stride,
                                        const int* seq_rows, const int* token_seq, const int* positions, void* out,
                                        int tokens, int hq, int hkv, int d, int dv, int page_size, float scale, int window,
                                        int num_pages, int* error, float softcap, int sink, const void* gate, int gate_pitch,
                                        const float* sink_logits, int keep_first, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (softcap < 0.f || (gate != nullptr && gate_pitch < hq * dv) || keep_first < 0) return SE_ERR_ARGUMENT;
    if (sink_logits != nullptr) sink = 1;
    if (d > 32 * se::kMaxDimPerLane || d <= 0 || dv > 32 * se::kMaxDimPerLane || dv <= 0 || hkv <= 0 || hq % hkv)
        return SE_ERR_UNSUPPORTED;
    dim3 grid(tokens, hq);
    SE_DISPATCH_DTYPE(dtype, T,
        se::paged_attention_plain_kernel<T><<<grid, 32 * se::kAttnWarps, 0, stream>>>(
            (const T*)q, (const T*)cache, table, table_stride, seq_rows, token_seq, positions, (T*)out, hq, hkv, d, dv,
            page_size, scale, window, num_pages, error, softcap, sink, (const T*)gate, gate_pitch,
            sink_logits, keep_first));
    SE_LAUNCH_CHECK();
}
