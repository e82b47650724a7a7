// Several copies of the residual stream ("streams") in place of one. A sublayer reads a weighted sum of the copies,
//
//     u = sum_s a[s] X[s],      xn = w * u / sqrt(mean(u^2) + eps)        (w: the norm's weight, offset included)
//
// and its result y rewrites every copy at once from the old ones,
//
//     X'[t] = sum_s M[s, t] X[s] + b[t] y.
//
// One kernel does, per token row, any of: the rewrite by the sublayer that just ran (y given), the read of the
// sublayer that runs next (a given), and the sum of the copies (where a single stream is wanted again: a tap, the
// model's last norm). X is [T, S, D] 32-bit; a row's S copies lie behind one another. Everything is 32-bit; the
// sums over the copies run in the copies' order, the row's sum of squares is each thread's chain over its pieces,
// added by a fixed xor tree and then over the warps in index order: a row's result depends on that row only.
#include "common.cuh"

namespace gi {

constexpr int kMaxStreams = 8;
constexpr int kStreamsKept = 4;        // pieces of u that a thread keeps in registers between the two passes

template <int VEC> struct Vals { float v[VEC]; };
template <int VEC> __device__ __forceinline__ Vals<VEC> load_vals(const float* p) {
    Vals<VEC> r;
    if constexpr (VEC == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
    else r.v[0] = *p;
    return r;
}
template <int VEC> __device__ __forceinline__ void store_vals(float* p, const Vals<VEC>& r) {
    if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    else *p = r.v[0];
}
template <int VEC, typename TOut> __device__ __forceinline__ void store_vals_as(TOut* p, const Vals<VEC>& r) {
    if constexpr (VEC == 4 && sizeof(TOut) == 2) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[1]), hi = __floats2bfloat162_rn(r.v[2], r.v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&lo); raw.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = raw;
    } else if constexpr (VEC == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    } else {
        *p = from_float<TOut>(r.v[0]);
    }
}

struct StreamsArgs {
    float* X;                  // [T, S, D]
    const float* single;       // [T, D] or null: the copies are all this row (the model's start); X is written from it
    float* y;                  // [T, D] or null: the sublayer's result; with it the copies are rewritten
    int clear_y;               // y = 0 afterwards (the next sublayer adds into it)
    const float* mix;          // [S, S], indexed [from, to]
    const float* out_w;        // [S]
    const float* in_w;         // [S] or null: the next sublayer's read
    const float* norm_w;       // [D], with in_w
    float eps;
    void* xn_out;              // [T, D], with in_w
    float* sum_out;            // [T, D] or null
    int S, D;
};

template <typename TOut, int VEC, int NS>
__global__ void __launch_bounds__(256)
streams_kernel(const StreamsArgs p) {
    pdl_prologue();
    __shared__ float warp_part[8];
    __shared__ float s_mix[kMaxStreams * kMaxStreams], s_out[kMaxStreams], s_in[kMaxStreams];
    const int S = NS ? NS : p.S, D = p.D;
    if (threadIdx.x < S * S && p.y) s_mix[threadIdx.x] = p.mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (p.y) s_out[threadIdx.x] = p.out_w[threadIdx.x];
        if (p.in_w) s_in[threadIdx.x] = p.in_w[threadIdx.x];
    }
    __syncthreads();
    const size_t row = static_cast<size_t>(blockIdx.x);
    float* X = p.X + row * S * D;
    constexpr int kS = NS ? NS : kMaxStreams;
    // pieces whose reads are all requested before anything of them is written (fewer with more copies: registers)
    constexpr int kBatch = kS <= 2 ? 4 : kS <= 4 ? 2 : 1;
    float ss = 0.f;

    struct In { Vals<VEC> old[kS], yy; };
    auto read = [&](int d, In& in) {
#pragma unroll
        for (int s = 0; s < kS; ++s)
            if (s < S) in.old[s] = p.single ? (s == 0 ? load_vals<VEC>(p.single + row * D + d) : in.old[0])
                                            : load_vals<VEC>(X + static_cast<size_t>(s) * D + d);
        if (p.y) in.yy = load_vals<VEC>(p.y + row * D + d);
    };
    // rewrites the copies of one piece and returns the next sublayer's u
    auto write = [&](int d, const In& in) -> Vals<VEC> {
        Vals<VEC> u, sum;
        if (p.y && p.clear_y) {
            Vals<VEC> zero;
#pragma unroll
            for (int e = 0; e < VEC; ++e) zero.v[e] = 0.f;
            store_vals<VEC>(p.y + row * D + d, zero);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) u.v[e] = sum.v[e] = 0.f;
#pragma unroll
        for (int t = 0; t < kS; ++t) {
            if (t >= S) continue;
            Vals<VEC> nw = in.old[t];
            if (p.y) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) nw.v[e] = 0.f;
#pragma unroll
                for (int s = 0; s < kS; ++s) {
                    if (s >= S) continue;
                    const float m = s_mix[s * S + t];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) nw.v[e] = fmaf(m, in.old[s].v[e], nw.v[e]);
                }
#pragma unroll
                for (int e = 0; e < VEC; ++e) nw.v[e] = fmaf(s_out[t], in.yy.v[e], nw.v[e]);
            }
            if (p.y || p.single) store_vals<VEC>(X + static_cast<size_t>(t) * D + d, nw);
            if (p.in_w) {
                const float a = s_in[t];
#pragma unroll
                for (int e = 0; e < VEC; ++e) u.v[e] = fmaf(a, nw.v[e], u.v[e]);
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) sum.v[e] += nw.v[e];
        }
        if (p.sum_out) store_vals<VEC>(p.sum_out + row * D + d, sum);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss = fmaf(u.v[e], u.v[e], ss);
        return u;
    };

    Vals<VEC> keep[kStreamsKept];
#pragma unroll
    for (int i0 = 0; i0 < kStreamsKept; i0 += kBatch) {
        In in[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int d = ((i0 + b) * 256 + threadIdx.x) * VEC;
            if (d < D) read(d, in[b]);
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int d = ((i0 + b) * 256 + threadIdx.x) * VEC;
            if (d < D) keep[i0 + b] = write(d, in[b]);
        }
    }
    for (int d = (kStreamsKept * 256 + threadIdx.x) * VEC; d < D; d += 256 * VEC) {
        In in;
        read(d, in);
        write(d, in);
    }
    if (p.in_w == nullptr) return;
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += warp_part[k];
    const float scale = 1.0f / sqrtf(total / static_cast<float>(D) + p.eps);
    TOut* xn = static_cast<TOut*>(p.xn_out) + row * D;
    auto emit = [&](int d, const Vals<VEC>& u) {
        const Vals<VEC> w = load_vals<VEC>(p.norm_w + d);
        Vals<VEC> o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.v[e] = w.v[e] * (scale * u.v[e]);
        store_vals_as<VEC, TOut>(xn + d, o);
    };
#pragma unroll
    for (int i = 0; i < kStreamsKept; ++i) {
        const int d = (i * 256 + threadIdx.x) * VEC;
        if (d < D) emit(d, keep[i]);
    }
    // wider rows: u again from the copies as they now stand, in the same order
    for (int d = (kStreamsKept * 256 + threadIdx.x) * VEC; d < D; d += 256 * VEC) {
        Vals<VEC> u;
#pragma unroll
        for (int e = 0; e < VEC; ++e) u.v[e] = 0.f;
        for (int t = 0; t < S; ++t) {
            const Vals<VEC> nw = load_vals<VEC>(X + static_cast<size_t>(t) * D + d);
#pragma unroll
            for (int e = 0; e < VEC; ++e) u.v[e] = fmaf(s_in[t], nw.v[e], u.v[e]);
        }
        emit(d, u);
    }
}

}  // namespace gi

using namespace gi;

template <typename TOut, int VEC>
static void launch_streams(const StreamsArgs& a, int T, cudaStream_t st) {
    switch (a.S) {
        case 1: launch_kernel((streams_kernel<TOut, VEC, 1>), dim3(T), dim3(256), 0, st, a); break;
        case 2: launch_kernel((streams_kernel<TOut, VEC, 2>), dim3(T), dim3(256), 0, st, a); break;
        case 4: launch_kernel((streams_kernel<TOut, VEC, 4>), dim3(T), dim3(256), 0, st, a); break;
        default: launch_kernel((streams_kernel<TOut, VEC, 0>), dim3(T), dim3(256), 0, st, a); break;
    }
}

static int gi_streams_impl(float* X, const float* single, float* y, int clear_y, const float* mix, const float* out_w,
                           const float* in_w, const float* norm_w, float eps, void* xn_out, int xn_dtype, float* sum_out,
                           int T, int S, int D, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && D > 0, "streams: sizes must be positive");
    GI_REQUIRE(S >= 1 && S <= kMaxStreams, "streams: %d copies of the stream are not supported (1 to %d)", S, kMaxStreams);
    GI_REQUIRE(y == nullptr || (mix != nullptr && out_w != nullptr), "streams: a rewrite needs its mixing matrix and output weights");
    GI_REQUIRE(in_w == nullptr || (norm_w != nullptr && xn_out != nullptr), "streams: a read needs the norm's weight and an output");
    GI_REQUIRE(xn_dtype == kBF16 || xn_dtype == kF32, "streams: unsupported dtype code %d", xn_dtype);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto aligned = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    const bool vec = D % 4 == 0 && aligned(X) && aligned(single) && aligned(y) && aligned(norm_w) && aligned(xn_out) && aligned(sum_out);
    StreamsArgs a{X, single, y, clear_y, mix, out_w, in_w, norm_w, eps, xn_out, sum_out, S, D};
    if (xn_dtype == kBF16 && vec) launch_streams<__nv_bfloat16, 4>(a, T, st);
    else if (xn_dtype == kBF16) launch_streams<__nv_bfloat16, 1>(a, T, st);
    else if (vec) launch_streams<float, 4>(a, T, st);
    else launch_streams<float, 1>(a, T, st);
    return check_launch("streams");
}

extern "C" int gi_streams(float* X, const float* single, float* y, int clear_y, const float* mix, const float* out_w,
                          const float* in_w, const float* norm_w, float eps, void* xn_out, int xn_dtype, float* sum_out,
                          int T, int S, int D, void* stream) {
    return gi::dispatch(gi_streams_impl, X, single, y, clear_y, mix, out_w, in_w, norm_w, eps, xn_out, xn_dtype, sum_out, T, S, D, stream);
}
