// hyper_norm.cu -- the residual path of a decoder whose residual is kept in fp32 and may be several parallel streams
// ("hyper-connections"), fused with the pre-norm that follows it:
//
//   b2_embed_streams   x[t, s, :] = embed[token[t], :] * scale                      for every stream s
//   b2_hc_step         (1) when y is given: the streams are remixed and the sublayer output is written back,
//                              x'[t, j, :] = sum_s mix[s, j] * x[t, s, :] + out_w[j] * y[t, :]
//                      (2) when h is given: the next sublayer's input is read out and normalised,
//                              u = sum_s in_w[s] * x'[t, s, :];   h = norm(u) * w
//                          norm = layer norm without bias (B2_NORM_LAYER) or RMS norm (B2_NORM_RMS), eps inside the root.
//                      One pass over the streams does both: the sublayer's write-back and the next read-out touch the
//                      same fp32 rows, which is the only HBM traffic of the op (S*D*4 read + S*D*4 write + D out).
//                      S = 1 with mix = out_w = in_w = 1 is the ordinary residual add + norm.
// The streams and all statistics are fp32 whatever the activation type.
#include "b2_act.cuh"

namespace {

constexpr int kMaxStreams = 16;

template <typename T>
__global__ void embed_streams_kernel(const T* __restrict__ embed, const int64_t* __restrict__ tokens, int D, int S,
                                     float scale, float* __restrict__ x) {
    const int t = blockIdx.x;
    const T* row = embed + (size_t)tokens[t] * D;
    float* xo = x + (size_t)t * S * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = b2::ld(row + d) * scale;
        for (int s = 0; s < S; ++s) xo[(size_t)s * D + d] = v;
    }
}

// MS: compile-time bound on the number of streams (register arrays of MS x 4 values; S <= MS)
template <typename T, int MS>
__global__ void __launch_bounds__(512) hc_step_kernel(float* __restrict__ x, int S, int D, const T* __restrict__ y, int64_t y_stride,
                               const float* __restrict__ mix, const float* __restrict__ out_w,
                               const float* __restrict__ in_w, const float* __restrict__ norm_w, float eps, int norm_kind,
                               T* __restrict__ h, int64_t h_stride) {
    extern __shared__ float u_sm[];                  // [D] read-out of this token
    __shared__ float red[33];
    __shared__ float c_mix[kMaxStreams * kMaxStreams], c_out[kMaxStreams], c_in[kMaxStreams];
    const int t = blockIdx.x;
    if (threadIdx.x < S * S) c_mix[threadIdx.x] = mix ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
    if (threadIdx.x < S) {
        c_out[threadIdx.x] = out_w ? out_w[threadIdx.x] : 1.f;
        c_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 1.f;
    }
    __syncthreads();
    float* xt = x + (size_t)t * S * D;
    float sum = 0.f;
    // four columns per thread and 16-byte accesses to the streams when the width allows it
    const int W = (D % 4 == 0) ? 4 : 1;
    for (int d = threadIdx.x * W; d < D; d += blockDim.x * W) {
        float xs[MS][4];
#pragma unroll
        for (int s = 0; s < MS; ++s) {
            if (s < S) {
                if (W == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(xt + (size_t)s * D + d);
                    xs[s][0] = v.x; xs[s][1] = v.y; xs[s][2] = v.z; xs[s][3] = v.w;
                } else {
                    xs[s][0] = xt[(size_t)s * D + d];
                    xs[s][1] = xs[s][2] = xs[s][3] = 0.f;
                }
            } else {
                xs[s][0] = xs[s][1] = xs[s][2] = xs[s][3] = 0.f;
            }
        }
        if (y) {
            float yv[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c = 0; c < W; ++c) yv[c] = b2::ld(y + (size_t)t * y_stride + d + c);
            float nx[MS][4];
#pragma unroll
            for (int j = 0; j < MS; ++j) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float a = 0.f;
                    if (j < S) {
#pragma unroll
                        for (int s = 0; s < MS; ++s)
                            if (s < S) a = fmaf(c_mix[s * S + j], xs[s][c], a);
                        a = fmaf(c_out[j], yv[c], a);
                    }
                    nx[j][c] = a;
                }
                if (j < S) {
                    if (W == 4) *reinterpret_cast<float4*>(xt + (size_t)j * D + d) = make_float4(nx[j][0], nx[j][1], nx[j][2], nx[j][3]);
                    else xt[(size_t)j * D + d] = nx[j][0];
                }
            }
#pragma unroll
            for (int j = 0; j < MS; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) xs[j][c] = nx[j][c];
        }
        if (h) {
            for (int c = 0; c < W; ++c) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < MS; ++s)
                    if (s < S) u = fmaf(c_in[s], xs[s][c], u);
                u_sm[d + c] = u;
                sum += u;
            }
        }
    }
    if (!h) return;
    __syncthreads();                                 // u_sm is read across threads from here on
    float mean = 0.f;
    if (norm_kind == B2_NORM_LAYER) mean = b2::block_sum(sum, red) / (float)D;
    float sq = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float c = u_sm[d] - mean;
        sq = fmaf(c, c, sq);
    }
    const float inv = rsqrtf(b2::block_sum(sq, red) / (float)D + eps);
    T* ho = h + (size_t)t * h_stride;
    for (int d = threadIdx.x; d < D; d += blockDim.x) b2::st(ho + d, (u_sm[d] - mean) * inv * norm_w[d]);
}

}  // namespace

extern "C" int b2_embed_streams(float* x, const void* embed, int act_dtype, const int64_t* tokens, int T, int D, int S,
                                float scale, void* stream) {
    B2_REQUIRE(T >= 0 && D > 0 && S >= 1 && S <= kMaxStreams, B2_EINVAL, "embed_streams: bad sizes T=%d D=%d S=%d", T, D, S);
    if (T == 0) return B2_OK;
    B2_REQUIRE(x && embed && tokens, B2_EINVAL, "embed_streams: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B2_DISPATCH_ACT(act_dtype, A, (embed_streams_kernel<A><<<T, 256, 0, st>>>(static_cast<const A*>(embed), tokens, D, S, scale, x)));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_hc_step(float* x, int T, int S, int D, const void* y, int64_t y_stride, const float* mix,
                          const float* out_w, const float* in_w, const float* norm_w, float eps, int norm_kind, void* h,
                          int64_t h_stride, int act_dtype, void* stream) {
    B2_REQUIRE(T >= 0 && D > 0 && S >= 1 && S <= kMaxStreams, B2_EINVAL, "hc_step: bad sizes T=%d D=%d S=%d", T, D, S);
    if (T == 0 || (!y && !h)) return B2_OK;
    B2_REQUIRE(x, B2_EINVAL, "hc_step: null streams");
    B2_REQUIRE(!h || norm_w, B2_EINVAL, "hc_step: a read-out needs the norm weight");
    B2_REQUIRE(norm_kind == B2_NORM_LAYER || norm_kind == B2_NORM_RMS, B2_EINVAL, "hc_step: unknown norm kind %d", norm_kind);
    const size_t smem = h ? (size_t)D * sizeof(float) : 0;
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "hc_step: width %d does not fit shared memory", D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int threads = D >= 4096 ? 512 : 256;
#define B2_HC(MS)                                                                                                          \
    do {                                                                                                                   \
        auto kern = hc_step_kernel<A, MS>;                                                                                 \
        if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<T, threads, smem, st>>>(x, S, D, static_cast<const A*>(y), y_stride, mix, out_w, in_w, norm_w, eps, norm_kind, \
                                       static_cast<A*>(h), h_stride);                                                      \
    } while (0)
    B2_DISPATCH_ACT(act_dtype, A, {
        if (S == 1) B2_HC(1);
        else if (S == 2) B2_HC(2);
        else if (S <= 4) B2_HC(4);
        else if (S <= 8) B2_HC(8);
        else B2_HC(16);
    });
#undef B2_HC
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
