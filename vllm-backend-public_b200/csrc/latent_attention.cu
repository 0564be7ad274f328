// latent_attention.cu -- softmax attention whose keys and values are rebuilt from ONE low-rank latent per token that all
// heads share, plus one rotated key part that all heads share as well.  Per token the paged pool keeps a row
//   cache [num_blocks, bs, R + dr] = [ latent c (R, RMS-normed) | rotated key part (dr) ]        (activation type)
// and nothing per head.  With per-head up-projections K_h = W_uk[h] c and V_h = W_uv[h] c the score of head h is
//   s = scale * ( (W_uk[h]^T q_h) . c  +  q_rot_h . k_rot ),
// so a query that has been carried into the latent space ("absorbed": qa_h = [ W_uk[h]^T q_h | q_rot_h ], size R + dr) scores
// straight against the cache rows, and the head's output is W_uv[h] applied to sum_j p_j c_j.  Every head reads the same
// R + dr numbers per key: the op is multi-query attention with key size R + dr and value = the first R entries of the key.
//
//   b2_latent_prep        per token: the rotated parts of the query heads are rotated (pairs 2i, 2i+1 of the first
//                         `rot_dims` entries; angle and magnitude from a fp32 table [max_pos, rot_dims] = cos | sin halves)
//                         and written behind the absorbed part of qa; when the layer owns a down-projection its first R
//                         outputs are RMS-normed (plain weight) into the cache row at the token's slot and the last dr,
//                         rotated, behind them.  A layer that reads another layer's pool passes dkv_off < 0.
//   b2_latent_attention   o[t, h, :R] = gate[t, h] * sum_j softmax_j(s)[j] c_j over the visible keys: j <= i, and with a
//                         window W > 0 also i - j < W.  gate = sigmoid of a per-head column of the projection rows
//                         (gate NULL: 1).  Softmax state, scores and the accumulator are fp32.
// Sequences are described like everywhere in this library: rows cu_q[i] .. cu_q[i+1]-1, ctx_start[i] cached tokens before
// them (< 0: padding, output rows are zeroed), block_tables[i, :].
#include "b2_act.cuh"

namespace {

constexpr int kMaxRPerLane = 16;                     // R <= 512 in the warp kernel

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int64_t proj_stride, int H, int dn, int dr, int rot_dims, int R,
                                   int q_off, int dkv_off, const float* __restrict__ norm_w, float eps,
                                   const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, int max_pos,
                                   const int64_t* __restrict__ slots, int bs, T* __restrict__ qa, T* __restrict__ cache) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * proj_stride;
    const int Dc = R + dr, half = rot_dims / 2;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + (size_t)pos * rot_dims;
    // query heads: [dn | dr] -> the dr part, rotated, behind the R absorbed entries of qa[t, h]
    for (int idx = threadIdx.x; idx < H * dr; idx += blockDim.x) {
        const int hh = idx / dr, i = idx % dr;
        const T* src = row + q_off + (size_t)hh * (dn + dr) + dn;
        float v = b2::ld(src + i);
        if (i < rot_dims) {
            const int pr = i >> 1;
            const float c = cs[pr], s = cs[half + pr];
            const float other = b2::ld(src + (i ^ 1));
            v = (i & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
        }
        b2::st(qa + ((size_t)t * H + hh) * Dc + R + i, v);
    }
    if (dkv_off < 0) return;
    const int64_t slot = slots[t];
    if (slot < 0) return;                            // uniform over the block
    T* dst = cache + (size_t)slot * Dc;
    const T* src = row + dkv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = b2::ld(src + i);
        ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(b2::block_sum(ss, red) / (float)R + eps);
    for (int i = threadIdx.x; i < R; i += blockDim.x) b2::st(dst + i, b2::ld(src + i) * inv * (norm_w ? norm_w[i] : 1.f));
    for (int i = threadIdx.x; i < dr; i += blockDim.x) {
        float v = b2::ld(src + R + i);
        if (i < rot_dims) {
            const int pr = i >> 1;
            const float c = cs[pr], s = cs[half + pr];
            const float other = b2::ld(src + R + (i ^ 1));
            v = (i & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
        }
        b2::st(dst + R + i, v);
    }
}

// One warp per (row, head): scores of 32 keys at a time (a lane per key), online softmax, P.C with a lane per latent column.
// Any sizes, both activation types; the tensor-core kernel below takes the bf16 shapes it is built for.
template <typename T>
__global__ void latent_attention_kernel(const T* __restrict__ qa, const T* __restrict__ cache,
                                        const int32_t* __restrict__ block_tables, int max_nb, const int32_t* __restrict__ cu_q,
                                        const int32_t* __restrict__ ctx_start, int n_seq, int rows, int H, int R, int dr, int bs,
                                        float scale, int window, const T* __restrict__ gate, int64_t gate_stride,
                                        T* __restrict__ out) {
    extern __shared__ float q_sm[];                  // [warps, R + dr]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int item = blockIdx.x * (blockDim.x >> 5) + wid;       // (row, head)
    if (item >= rows * H) return;
    const int row = item / H, hh = item % H;
    const int seq = b2::seq_of_row(cu_q, n_seq, row);
    const int ctx = ctx_start[seq];
    const int Dc = R + dr;
    T* dst = out + (size_t)item * R;
    if (ctx < 0) {
        for (int i = lane; i < R; i += 32) b2::st(dst + i, 0.f);
        return;
    }
    const int pos = ctx + row - cu_q[seq];
    const int lo = window > 0 ? max(pos - window + 1, 0) : 0;
    float* qs = q_sm + (size_t)wid * Dc;
    const T* qv = qa + (size_t)item * Dc;
    for (int i = lane; i < Dc; i += 32) qs[i] = b2::ld(qv + i) * scale;
    __syncwarp();
    const int32_t* bt = block_tables + (size_t)seq * max_nb;
    float m = -INFINITY, l = 0.f;
    float acc[kMaxRPerLane];
#pragma unroll
    for (int c = 0; c < kMaxRPerLane; ++c) acc[c] = 0.f;
    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        size_t base = 0;
        if (j <= pos) {
            base = ((size_t)bt[j / bs] * bs + (j % bs)) * Dc;
            const T* kr = cache + base;
            float d0 = 0.f, d1 = 0.f;
            int i = 0;
            for (; i + 1 < Dc; i += 2) {
                d0 = fmaf(qs[i], b2::ld(kr + i), d0);
                d1 = fmaf(qs[i + 1], b2::ld(kr + i + 1), d1);
            }
            if (i < Dc) d0 = fmaf(qs[i], b2::ld(kr + i), d0);
            s = d0 + d1;
        }
        const float m_new = fmaxf(m, b2::warp_max(s));
        const float corr = m == -INFINITY ? 0.f : __expf(m - m_new);
        const float p = j <= pos ? __expf(s - m_new) : 0.f;
        l = l * corr + b2::warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < kMaxRPerLane; ++c) acc[c] *= corr;
        const int nk = min(32, pos - j0 + 1);
        for (int kk = 0; kk < nk; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const size_t vb = __shfl_sync(0xffffffffu, (unsigned long long)base, kk);
            const T* vr = cache + vb;
#pragma unroll
            for (int c = 0; c < kMaxRPerLane; ++c) {
                const int i = lane + 32 * c;
                if (i < R) acc[c] = fmaf(pk, b2::ld(vr + i), acc[c]);
            }
        }
    }
    float f = l > 0.f ? 1.f / l : 0.f;
    if (gate) f *= b2::sigmoid_f(b2::ld(gate + (size_t)row * gate_stride + hh));
#pragma unroll
    for (int c = 0; c < kMaxRPerLane; ++c) {
        const int i = lane + 32 * c;
        if (i < R) b2::st(dst + i, acc[c] * f);
    }
}

}  // namespace

extern "C" int b2_latent_prep(const void* proj, int64_t proj_stride, int act_dtype, int T, int H, int dn, int dr, int rot_dims,
                              int R, int q_off, int dkv_off, const float* norm_w, float eps, const int32_t* positions,
                              const float* cos_sin, int max_pos, const int64_t* slots, int bs, void* qa, void* cache,
                              void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && dn >= 0 && dr >= 0 && R > 0 && bs > 0 && q_off >= 0 && rot_dims >= 0 && rot_dims <= dr &&
                   rot_dims % 2 == 0 && max_pos > 0, B2_EINVAL, "latent_prep: bad sizes");
    if (T == 0) return B2_OK;
    B2_REQUIRE(proj && positions && qa && (rot_dims == 0 || cos_sin), B2_EINVAL, "latent_prep: null pointer");
    B2_REQUIRE(dkv_off < 0 || (slots && cache), B2_EINVAL, "latent_prep: a layer with a down-projection needs slots and its pool");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int work = H * dr > R ? H * dr : R;
    const int threads = work >= 512 ? 256 : 128;
    B2_DISPATCH_ACT(act_dtype, A, (latent_prep_kernel<A><<<T, threads, 0, st>>>(
        static_cast<const A*>(proj), proj_stride, H, dn, dr, rot_dims, R, q_off, dkv_off, norm_w, eps, positions, cos_sin, max_pos,
        slots, bs, static_cast<A*>(qa), static_cast<A*>(cache))));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_latent_attention(void* out, const void* qa, const void* cache, int act_dtype, const int32_t* block_tables,
                                   int max_nb, const int32_t* cu_q, const int32_t* ctx_start, int n_seq, int T, int H, int R,
                                   int dr, int bs, float scale, int window, const void* gate, int64_t gate_stride,
                                   void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && R > 0 && dr >= 0 && bs > 0 && window >= 0, B2_EINVAL, "latent_attention: bad sizes");
    B2_REQUIRE(R <= 32 * kMaxRPerLane, B2_EUNSUPPORTED, "latent_attention: latent size %d above %d", R, 32 * kMaxRPerLane);
    if (T == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(out && qa && cache && block_tables && cu_q && ctx_start, B2_EINVAL, "latent_attention: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps = 4;
    const size_t smem = (size_t)warps * (R + dr) * sizeof(float);
    B2_REQUIRE(smem <= 48 * 1024, B2_EUNSUPPORTED, "latent_attention: key size %d too large", R + dr);
    const int items = T * H, blocks = (items + warps - 1) / warps;
    B2_DISPATCH_ACT(act_dtype, A, (latent_attention_kernel<A><<<blocks, warps * 32, smem, st>>>(
        static_cast<const A*>(qa), static_cast<const A*>(cache), block_tables, max_nb, cu_q, ctx_start, n_seq, T, H, R, dr, bs,
        scale, window, static_cast<const A*>(gate), gate_stride, static_cast<A*>(out))));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
