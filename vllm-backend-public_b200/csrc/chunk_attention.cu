// chunk_attention.cu -- softmax attention without a rotation over a paged cache, with three parameters that other
// designs can set independently:
//   * per-head RMS norm of queries and keys (a plain weight of size dk shared by the heads),
//   * a block-local causal mask: position i sees j <= i with floor(j / chunk) == floor(i / chunk), blocks counted from
//     position 0 of the sequence (chunk = 0: plain causal),
//   * a sink: `sink` is added to the softmax denominator as exp(sink_logit - max), a key with no value (sink = 0: none;
//     sink = 1 with logit 0 gives p_j = exp(s_j) / (1 + sum exp(s))).
// Key size dk and value size dv are independent; K and V live in separate paged pools
//   k_cache [num_blocks, G, bs, dk],  v_cache [num_blocks, G, bs, dv]      (activation type).
//
//   b2_qknorm_cache      per token: q heads normalised into q_out; k heads normalised and written to the K pool, v copied
//                        to the V pool, through the token's slot (slot < 0 skips the write).
//   b2_chunk_attention   per (token, head) one warp: scores of 32 keys at a time (a lane per key), online softmax in fp32
//                        seeded with the sink, P.V with a lane per value column.  With the mask a query touches at most
//                        `chunk` keys wherever it stands, so prompt chunks and decode rows run the same kernel; a decode
//                        row is a sequence with one query.
// Sequences are described like everywhere in this library: rows cu_q[i] .. cu_q[i+1]-1, ctx_start[i] cached tokens
// before them (< 0: padding, output rows are zeroed), block_tables[i, :].
#include "b2_act.cuh"

namespace {

constexpr int kMaxDvPerLane = 8;                     // dv <= 256

template <typename T>
__global__ void qknorm_cache_kernel(const T* __restrict__ qkv, int64_t qkv_stride, int H, int G, int dk, int dv,
                                    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                    const int64_t* __restrict__ slots, int bs, T* __restrict__ q_out,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache) {
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const T* src = qkv + (size_t)row * qkv_stride;
    const int64_t slot = slots[row];
    const int64_t blk = slot >= 0 ? slot / bs : 0;
    const int off = slot >= 0 ? (int)(slot % bs) : 0;
    for (int hd = wid; hd < H + 2 * G; hd += nw) {
        if (hd < H + G) {                            // q or k head: x / sqrt(mean(x^2) + eps) * w
            const T* v = src + (size_t)hd * dk;
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) {
                const float x = b2::ld(v + i);
                ss = fmaf(x, x, ss);
            }
            const float inv = rsqrtf(b2::warp_sum(ss) / (float)dk + eps);
            T* dst;
            const float* w;
            if (hd < H) {
                dst = q_out + ((size_t)row * H + hd) * dk;
                w = q_w;
            } else {
                if (slot < 0) continue;
                dst = k_cache + (((size_t)blk * G + (hd - H)) * bs + off) * dk;
                w = k_w;
            }
            for (int i = lane; i < dk; i += 32) b2::st(dst + i, b2::ld(v + i) * inv * (w ? w[i] : 1.f));
        } else {
            if (slot < 0) continue;
            const int g = hd - H - G;
            const T* v = src + (size_t)(H + G) * dk + (size_t)g * dv;
            T* dst = v_cache + (((size_t)blk * G + g) * bs + off) * dv;
            for (int i = lane; i < dv; i += 32) dst[i] = v[i];
        }
    }
}

template <typename T>
__global__ void chunk_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                       const int32_t* __restrict__ block_tables, int max_nb,
                                       const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start, int n_seq,
                                       int rows, int H, int G, int dk, int dv, int bs, float scale, int chunk, float sink,
                                       float sink_logit, T* __restrict__ out) {
    extern __shared__ float q_sm[];                  // [warps, dk]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int item = blockIdx.x * (blockDim.x >> 5) + wid;       // (row, head)
    if (item >= rows * H) return;
    const int row = item / H, hh = item % H;
    const int seq = b2::seq_of_row(cu_q, n_seq, row);
    const int ctx = ctx_start[seq];
    T* dst = out + (size_t)item * dv;
    if (ctx < 0) {
        for (int i = lane; i < dv; i += 32) b2::st(dst + i, 0.f);
        return;
    }
    const int pos = ctx + row - cu_q[seq];
    const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
    const int g = hh / (H / G);
    float* qs = q_sm + (size_t)wid * dk;
    const T* qv = q + (size_t)item * dk;
    for (int i = lane; i < dk; i += 32) qs[i] = b2::ld(qv + i) * scale;
    __syncwarp();
    const int32_t* bt = block_tables + (size_t)seq * max_nb;
    float m = sink > 0.f ? sink_logit : -INFINITY, l = sink;      // the sink seeds the running maximum and denominator
    float acc[kMaxDvPerLane];
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) acc[c] = 0.f;
    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        size_t vbase = 0;
        if (j <= pos) {
            const size_t tile = ((size_t)bt[j / bs] * G + g) * bs + (j % bs);
            const T* kr = k_cache + tile * dk;
            vbase = tile * dv;
            float d = 0.f;
            for (int i = 0; i < dk; ++i) d = fmaf(qs[i], b2::ld(kr + i), d);
            s = d;
        }
        const float m_new = fmaxf(m, b2::warp_max(s));
        const float corr = m == -INFINITY ? 0.f : __expf(m - m_new);
        const float p = j <= pos ? __expf(s - m_new) : 0.f;
        l = l * corr + b2::warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < kMaxDvPerLane; ++c) acc[c] *= corr;
        const int nk = min(32, pos - j0 + 1);
        for (int kk = 0; kk < nk; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const size_t vb = __shfl_sync(0xffffffffu, (unsigned long long)vbase, kk);
            const T* vr = v_cache + vb;
#pragma unroll
            for (int c = 0; c < kMaxDvPerLane; ++c) {
                const int i = lane + 32 * c;
                if (i < dv) acc[c] = fmaf(pk, b2::ld(vr + i), acc[c]);
            }
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) b2::st(dst + i, acc[c] * inv);
    }
}

}  // namespace

extern "C" int b2_qknorm_cache(const void* qkv, int64_t qkv_stride, int act_dtype, int T, int H, int G, int dk, int dv,
                               const float* q_w, const float* k_w, float eps, const int64_t* slots, int bs, void* q_out,
                               void* k_cache, void* v_cache, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && bs > 0, B2_EINVAL, "qknorm_cache: bad sizes");
    if (T == 0) return B2_OK;
    B2_REQUIRE(qkv && slots && q_out && k_cache && v_cache, B2_EINVAL, "qknorm_cache: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps = H + 2 * G < 8 ? H + 2 * G : 8;
    B2_DISPATCH_ACT(act_dtype, A, (qknorm_cache_kernel<A><<<T, warps * 32, 0, st>>>(
        static_cast<const A*>(qkv), qkv_stride, H, G, dk, dv, q_w, k_w, eps, slots, bs, static_cast<A*>(q_out),
        static_cast<A*>(k_cache), static_cast<A*>(v_cache))));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_chunk_attention(void* out, const void* q, const void* k_cache, const void* v_cache, int act_dtype,
                                  const int32_t* block_tables, int max_nb, const int32_t* cu_q, const int32_t* ctx_start,
                                  int n_seq, int T, int H, int G, int dk, int dv, int bs, float scale, int chunk, float sink,
                                  float sink_logit, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && bs > 0 && chunk >= 0 && sink >= 0.f, B2_EINVAL,
               "chunk_attention: bad sizes");
    B2_REQUIRE(dv <= 32 * kMaxDvPerLane, B2_EUNSUPPORTED, "chunk_attention: value size %d above %d", dv, 32 * kMaxDvPerLane);
    if (T == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(out && q && k_cache && v_cache && block_tables && cu_q && ctx_start, B2_EINVAL, "chunk_attention: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps = 4;
    const size_t smem = (size_t)warps * dk * sizeof(float);
    B2_REQUIRE(smem <= 48 * 1024, B2_EUNSUPPORTED, "chunk_attention: key size %d too large", dk);
    const int items = T * H, blocks = (items + warps - 1) / warps;
    B2_DISPATCH_ACT(act_dtype, A, (chunk_attention_kernel<A><<<blocks, warps * 32, smem, st>>>(
        static_cast<const A*>(q), static_cast<const A*>(k_cache), static_cast<const A*>(v_cache), block_tables, max_nb, cu_q,
        ctx_start, n_seq, T, H, G, dk, dv, bs, scale, chunk, sink, sink_logit, static_cast<A*>(out))));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
