// Kernels of layers whose mixer and feed-forward read one normed input and are added together, of a residual stream
// that is a weighted mix of all earlier layers' results, and a few small element-wise steps around them.
//
//   add_rows_at     x[t, :] += table[index[t], :]: a learned vector per position added to the embedding
//   add_bias        y[t, :] += b: the bias of a product that adds into a stream
//   sigmoid_gate    out[t, c] = a[t, c] * sigmoid(g[t, off + c]): an element-wise output gate (out in the compute dtype)
//   depth_mix       with h [T, slots, D] the results kept so far (slot 0 the embedding's output, slot i + 1 layer i's),
//                   x the stream that layer i read and y what its sublayers produced:
//                   h[t, i + 1] = x[t] + m (y[t] + b);  x[t] = sum_{j <= i + 1} w[j] h[t, j]   (w: the layer's i + 2 mixing
//                   weights; b: an optional bias that a sublayer's last product left to this kernel);
//                   without weights x[t] += m (y[t] + b). The same pass clears y and writes the unit-RMS norm of the new x
//                   times one number (the next layer's single norm weight) in the compute dtype.
//   softcap         z <- cap * tanh(z / cap), in place
//
// All arithmetic is 32-bit; only stores to a bfloat16 output round. A row's result depends on that row only.
#include "common.cuh"

namespace gi {

template <typename TTab>
__global__ void __launch_bounds__(256)
add_rows_at_kernel(float* __restrict__ x, const TTab* __restrict__ table, const int* __restrict__ index, int D, int table_rows,
                   size_t total) {
    pdl_prologue();
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256) {
        const size_t t = i / D;
        const int d = static_cast<int>(i % D);
        int r = index[t];
        r = r < 0 ? 0 : (r >= table_rows ? table_rows - 1 : r);       // the host refuses positions outside the table
        x[i] += to_float(table[static_cast<size_t>(r) * D + d]);
    }
}

__global__ void __launch_bounds__(256)
add_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, int D, size_t total) {
    pdl_prologue();
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256)
        y[i] += bias[i % D];
}

template <typename TOut>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const float* __restrict__ a, const float* __restrict__ g, long long ldg, int g_off, TOut* __restrict__ out, int N,
                    size_t total) {
    pdl_prologue();
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256) {
        const size_t t = i / N;
        const int c = static_cast<int>(i % N);
        const float z = g[t * ldg + g_off + c];
        out[i] = from_float<TOut>(a[i] * (1.0f / (1.0f + expf(-z))));
    }
}

__global__ void __launch_bounds__(256)
softcap_kernel(float* __restrict__ z, float cap, float inv_cap, size_t total) {
    pdl_prologue();
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256)
        z[i] = cap * tanhf(z[i] * inv_cap);
}

__global__ void __launch_bounds__(256)
scale_kernel(float* __restrict__ z, float factor, size_t total) {
    pdl_prologue();
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256)
        z[i] *= factor;
}

constexpr int kDepthKept = 4;          // pieces of a row that a thread keeps in registers between the two passes
constexpr int kDepthWeights = 64;      // mixing weights held in shared memory (more are read from global memory)

template <int VEC> struct Piece { float v[VEC]; };
template <int VEC> __device__ __forceinline__ Piece<VEC> load_piece(const float* p) {
    Piece<VEC> r;
    if constexpr (VEC == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
    else r.v[0] = *p;
    return r;
}
template <int VEC> __device__ __forceinline__ void store_piece(float* p, const Piece<VEC>& r) {
    if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    else *p = r.v[0];
}
template <int VEC, typename TOut> __device__ __forceinline__ void store_piece_as(TOut* p, const Piece<VEC>& r) {
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

// One block per row; a thread takes pieces of VEC consecutive values (16-byte accesses when the width allows), piece
// i of thread t at (i * 256 + t) * VEC. The sum over the slots runs in slot order; the row's sum of squares is each
// thread's chain over its pieces, added by a fixed xor tree and then over the warps in index order: a row's result
// depends on that row only. The first kDepthKept pieces of a thread stay in registers for the second pass.
template <typename TOut, int VEC>
__global__ void __launch_bounds__(256)
depth_mix_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ y_bias, float m, float* __restrict__ hist, int slots, int slot,
                 const float* __restrict__ w, int first, const float* __restrict__ next_weight, float eps,
                 TOut* __restrict__ xn_out, int D) {
    pdl_prologue();
    __shared__ float warp_part[8];
    __shared__ float s_w[kDepthWeights];
    const size_t row = static_cast<size_t>(blockIdx.x) * D;
    float* h = hist ? hist + static_cast<size_t>(blockIdx.x) * slots * D : nullptr;
    if (h) {
        for (int j = threadIdx.x; j <= slot && j < kDepthWeights; j += 256) s_w[j] = w[j];
        __syncthreads();
    }
    Piece<VEC> keep[kDepthKept];
    float ss = 0.f;

    // what a piece reads: the stream, the sublayers' sum (with the bias) and the weighted sum of the kept results before
    // this layer's, in slot order (slot 0 is the stream itself while the history is still empty)
    auto read = [&](int d, Piece<VEC>& x_old, Piece<VEC>& yy, Piece<VEC>& acc) {
        x_old = load_piece<VEC>(x + row + d);
        yy = load_piece<VEC>(y + row + d);
        if (y_bias) {
            const Piece<VEC> b = load_piece<VEC>(y_bias + d);
#pragma unroll
            for (int e = 0; e < VEC; ++e) yy.v[e] += b.v[e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc.v[e] = 0.f;
        if (h) {
            for (int j = 0; j < slot; ++j) {
                const Piece<VEC> hj = (first && j == 0) ? x_old : load_piece<VEC>(h + static_cast<size_t>(j) * D + d);
                const float wj = j < kDepthWeights ? s_w[j] : w[j];
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc.v[e] = fmaf(wj, hj.v[e], acc.v[e]);
            }
        }
    };
    // what it writes, after all of a thread's reads are on their way: the layer's result into its slot, the mixed stream, y = 0
    auto write = [&](int d, const Piece<VEC>& x_old, const Piece<VEC>& yy, const Piece<VEC>& acc) -> Piece<VEC> {
        Piece<VEC> fresh, v, zero;
#pragma unroll
        for (int e = 0; e < VEC; ++e) { fresh.v[e] = x_old.v[e] + m * yy.v[e]; zero.v[e] = 0.f; }
        store_piece<VEC>(y + row + d, zero);
        v = fresh;
        if (h) {
            if (first) store_piece<VEC>(h + d, x_old);                  // slot 0: what the first layer read
            store_piece<VEC>(h + static_cast<size_t>(slot) * D + d, fresh);
            const float ws = slot < kDepthWeights ? s_w[slot] : w[slot];
#pragma unroll
            for (int e = 0; e < VEC; ++e) v.v[e] = fmaf(ws, fresh.v[e], acc.v[e]);
        }
        store_piece<VEC>(x + row + d, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss = fmaf(v.v[e], v.v[e], ss);
        return v;
    };

    {
        Piece<VEC> xo[kDepthKept], yy[kDepthKept], acc[kDepthKept];
#pragma unroll
        for (int i = 0; i < kDepthKept; ++i) {
            const int d = (i * 256 + threadIdx.x) * VEC;
            if (d < D) read(d, xo[i], yy[i], acc[i]);
        }
#pragma unroll
        for (int i = 0; i < kDepthKept; ++i) {
            const int d = (i * 256 + threadIdx.x) * VEC;
            if (d < D) keep[i] = write(d, xo[i], yy[i], acc[i]);
        }
    }
    for (int d = (kDepthKept * 256 + threadIdx.x) * VEC; d < D; d += 256 * VEC) {
        Piece<VEC> xo, yy, acc;
        read(d, xo, yy, acc);
        write(d, xo, yy, acc);
    }
    if (xn_out == nullptr) return;
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += warp_part[k];
    const float scale = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
    const float g = next_weight ? next_weight[0] : 1.0f;
#pragma unroll
    for (int i = 0; i < kDepthKept; ++i) {
        const int d = (i * 256 + threadIdx.x) * VEC;
        if (d < D) {
            Piece<VEC> o;
#pragma unroll
            for (int e = 0; e < VEC; ++e) o.v[e] = g * (scale * keep[i].v[e]);
            store_piece_as<VEC, TOut>(xn_out + row + d, o);
        }
    }
    for (int d = (kDepthKept * 256 + threadIdx.x) * VEC; d < D; d += 256 * VEC) {
        Piece<VEC> o = load_piece<VEC>(x + row + d);
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.v[e] = g * (scale * o.v[e]);
        store_piece_as<VEC, TOut>(xn_out + row + d, o);
    }
}

}  // namespace gi

using namespace gi;

static unsigned grid_for(size_t total) { return static_cast<unsigned>(std::min<size_t>((total + 255) / 256, 148 * 16)); }

static int gi_add_rows_at_impl(float* x, const void* table, int table_dtype, const int* index, int T, int D, int table_rows, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && D > 0 && table_rows > 0, "add_rows_at: sizes must be positive");
    const size_t total = static_cast<size_t>(T) * D;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (table_dtype == kBF16)
        launch_kernel((add_rows_at_kernel<__nv_bfloat16>), dim3(grid_for(total)), dim3(256), 0, st, x, static_cast<const __nv_bfloat16*>(table), index, D, table_rows, total);
    else if (table_dtype == kF32)
        launch_kernel((add_rows_at_kernel<float>), dim3(grid_for(total)), dim3(256), 0, st, x, static_cast<const float*>(table), index, D, table_rows, total);
    else
        GI_REQUIRE(false, "add_rows_at: unsupported dtype code %d", table_dtype);
    return check_launch("add_rows_at");
}

static int gi_add_bias_impl(float* y, const float* bias, int T, int D, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && D > 0, "add_bias: sizes must be positive");
    const size_t total = static_cast<size_t>(T) * D;
    launch_kernel(add_bias_kernel, dim3(grid_for(total)), dim3(256), 0, static_cast<cudaStream_t>(stream), y, bias, D, total);
    return check_launch("add_bias");
}

static int gi_sigmoid_gate_impl(const float* a, const float* g, long long ldg, int g_off, void* out, int out_dtype, int T, int N, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && N > 0 && g_off >= 0 && g_off + N <= ldg, "sigmoid_gate: the gate's columns lie outside its rows");
    const size_t total = static_cast<size_t>(T) * N;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == kBF16)
        launch_kernel((sigmoid_gate_kernel<__nv_bfloat16>), dim3(grid_for(total)), dim3(256), 0, st, a, g, ldg, g_off, static_cast<__nv_bfloat16*>(out), N, total);
    else if (out_dtype == kF32)
        launch_kernel((sigmoid_gate_kernel<float>), dim3(grid_for(total)), dim3(256), 0, st, a, g, ldg, g_off, static_cast<float*>(out), N, total);
    else
        GI_REQUIRE(false, "sigmoid_gate: unsupported dtype code %d", out_dtype);
    return check_launch("sigmoid_gate");
}

static int gi_softcap_impl(float* z, long long total, float cap, void* stream) {
    if (total == 0) return 0;
    GI_REQUIRE(total > 0 && cap > 0.f, "softcap: the size and the cap must be positive");
    launch_kernel(softcap_kernel, dim3(grid_for(static_cast<size_t>(total))), dim3(256), 0, static_cast<cudaStream_t>(stream), z, cap, 1.0f / cap,
                  static_cast<size_t>(total));
    return check_launch("softcap");
}

static int gi_scale_impl(float* z, long long total, float factor, void* stream) {
    if (total == 0) return 0;
    GI_REQUIRE(total > 0, "scale: the size must be positive");
    launch_kernel(scale_kernel, dim3(grid_for(static_cast<size_t>(total))), dim3(256), 0, static_cast<cudaStream_t>(stream), z, factor,
                  static_cast<size_t>(total));
    return check_launch("scale");
}

static int gi_depth_mix_impl(float* x, float* y, const float* y_bias, float m, float* hist, int slots, int slot, const float* w, int first,
                             const float* next_weight, float eps, void* xn_out, int xn_dtype, int T, int D, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && D > 0, "depth_mix: sizes must be positive");
    GI_REQUIRE(hist == nullptr || (w != nullptr && slot >= 1 && slot < slots), "depth_mix: slot %d lies outside the %d kept results", slot, slots);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec = D % 4 == 0 && aligned(x) && aligned(y) && aligned(hist) && aligned(y_bias) && aligned(xn_out);
    GI_REQUIRE(xn_dtype == kBF16 || xn_dtype == kF32, "depth_mix: unsupported dtype code %d", xn_dtype);
    if (xn_dtype == kBF16 && vec)
        launch_kernel((depth_mix_kernel<__nv_bfloat16, 4>), dim3(T), dim3(256), 0, st, x, y, y_bias, m, hist, slots, slot, w, first, next_weight, eps,
                      static_cast<__nv_bfloat16*>(xn_out), D);
    else if (xn_dtype == kBF16)
        launch_kernel((depth_mix_kernel<__nv_bfloat16, 1>), dim3(T), dim3(256), 0, st, x, y, y_bias, m, hist, slots, slot, w, first, next_weight, eps,
                      static_cast<__nv_bfloat16*>(xn_out), D);
    else if (vec)
        launch_kernel((depth_mix_kernel<float, 4>), dim3(T), dim3(256), 0, st, x, y, y_bias, m, hist, slots, slot, w, first, next_weight, eps,
                      static_cast<float*>(xn_out), D);
    else
        launch_kernel((depth_mix_kernel<float, 1>), dim3(T), dim3(256), 0, st, x, y, y_bias, m, hist, slots, slot, w, first, next_weight, eps,
                      static_cast<float*>(xn_out), D);
    return check_launch("depth_mix");
}

extern "C" int gi_add_rows_at(float* x, const void* table, int table_dtype, const int* index, int T, int D, int table_rows, void* stream) {
    return gi::dispatch(gi_add_rows_at_impl, x, table, table_dtype, index, T, D, table_rows, stream);
}

extern "C" int gi_add_bias(float* y, const float* bias, int T, int D, void* stream) {
    return gi::dispatch(gi_add_bias_impl, y, bias, T, D, stream);
}

extern "C" int gi_sigmoid_gate(const float* a, const float* g, long long ldg, int g_off, void* out, int out_dtype, int T, int N, void* stream) {
    return gi::dispatch(gi_sigmoid_gate_impl, a, g, ldg, g_off, out, out_dtype, T, N, stream);
}

extern "C" int gi_softcap(float* z, long long total, float cap, void* stream) {
    return gi::dispatch(gi_softcap_impl, z, total, cap, stream);
}

extern "C" int gi_scale(float* z, long long total, float factor, void* stream) {
    return gi::dispatch(gi_scale_impl, z, total, factor, stream);
}

extern "C" int gi_depth_mix(float* x, float* y, const float* y_bias, float m, float* hist, int slots, int slot, const float* w, int first,
                            const float* next_weight, float eps, void* xn_out, int xn_dtype, int T, int D, void* stream) {
    return gi::dispatch(gi_depth_mix_impl, x, y, y_bias, m, hist, slots, slot, w, first, next_weight, eps, xn_out, xn_dtype, T, D, stream);
}
