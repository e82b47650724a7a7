// Kernels of layers that normalise after the residual sum, of gated feed-forwards with other activations
// than SiLU, and of attention whose queries and keys are normalised per head before the rotation.
//
//   scale_cast      acc = alpha * x (32-bit) and xn = x in the compute dtype: what a sublayer of a post-norm layer
//                   reads (xn) and what it adds its output to (acc)
//   residual_norm   x = w * (acc / sqrt(mean(acc^2) + eps)) in 32-bit, in one pass also the next sublayer's
//                   xn = x (compute dtype) and acc = alpha * x
//   gated_act       out = act(gate) * up for act in {SiLU, ReLU, tanh-GELU, capped swish}, optionally with a bias on both
//   norm_rope_store per token and head: optional unit-RMS norm with a weight shared by all heads, rotation of the
//                   first 2 * rot_half dimensions by angles position * freq[i] computed here in 32-bit (no table
//                   of max_position rows), queries to q_out, keys to the token's page row; the values stored beside
//                   them come from any column of the same input row (the keys as projected, for a design whose
//                   values are its keys).
//
//   add_normed      x += w * (y / sqrt(mean(y^2) + eps)): a layer whose norm stands on the sublayer's output. The same
//                   pass leaves xn = x in the compute dtype (what the next sublayer reads) and clears y (what it
//                   adds its output to)
//   latent_store    per token, from one row of 32-bit projections: a query latent brought to unit RMS and weighted,
//                   to q_latent; a key/value latent likewise, into the first columns of the token's page row; a
//                   rotated part shared by all heads (angles position * freq[i], cos and sin times a constant) behind it
//
// All arithmetic is 32-bit; only stores round. A row's result depends on that row only.
#include "common.cuh"

namespace gi {

__device__ __forceinline__ float block_sum_256(float v, float* warp_part) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += warp_part[w];
    __syncthreads();
    return total;
}

template <typename TOut>
__global__ void __launch_bounds__(256)
scale_cast_kernel(const float* __restrict__ x, float* __restrict__ acc, TOut* __restrict__ xn, float alpha, size_t total) {
    pdl_prologue();
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256) {
        const float v = x[i];
        acc[i] = alpha * v;
        if (xn) xn[i] = from_float<TOut>(v);
    }
}

// One block per row; the row's sum of squares is taken by a fixed strided assignment, a fixed xor tree and the
// warps in index order (the order of the RMSNorm kernel), so a row never depends on the batch.
template <typename TOut>
__global__ void __launch_bounds__(256)
residual_norm_kernel(const float* __restrict__ acc_in, const float* __restrict__ weight, float* __restrict__ x_out,
                     float* __restrict__ acc_out, TOut* __restrict__ xn_out, int D, float eps, float alpha) {
    pdl_prologue();
    __shared__ float warp_part[8];
    const size_t row = static_cast<size_t>(blockIdx.x) * D;
    const float* a = acc_in + row;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += 256) ss = fmaf(a[d], a[d], ss);
    const float total = block_sum_256(ss, warp_part);
    const float scale = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
    for (int d = threadIdx.x; d < D; d += 256) {
        const float v = weight[d] * (scale * a[d]);
        x_out[row + d] = v;
        if (acc_out) acc_out[row + d] = alpha * v;
        if (xn_out) xn_out[row + d] = from_float<TOut>(v);
    }
}

template <typename TOut>
__global__ void __launch_bounds__(256)
gated_act_kernel(const float* __restrict__ gu, const float* __restrict__ bias, TOut* __restrict__ out, int I, size_t total, int act,
                 float limit) {
    pdl_prologue();
    const size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / I;
    const int c = static_cast<int>(i % I);
    float g = gu[t * 2 * I + c], u = gu[t * 2 * I + I + c];
    if (bias) { g += bias[c]; u += bias[I + c]; }
    out[i] = from_float<TOut>(gated_value(g, u, act, limit));
}

// The same, four channels to a thread with 16-byte accesses (I a multiple of 4, pointers aligned).
template <typename TOut>
__global__ void __launch_bounds__(256)
gated_act4_kernel(const float* __restrict__ gu, const float* __restrict__ bias, TOut* __restrict__ out, int I4, size_t total4, int act,
                  float limit) {
    pdl_prologue();
    const size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total4) return;
    const size_t t = i / I4;
    const int c = static_cast<int>(i % I4);
    const float4* row = reinterpret_cast<const float4*>(gu) + t * 2 * I4;
    float4 g = row[c], u = row[I4 + c];
    if (bias) {
        const float4 bg = reinterpret_cast<const float4*>(bias)[c], bu = reinterpret_cast<const float4*>(bias)[I4 + c];
        g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w;
        u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
    }
    const float r0 = gated_value(g.x, u.x, act, limit), r1 = gated_value(g.y, u.y, act, limit), r2 = gated_value(g.z, u.z, act, limit),
                r3 = gated_value(g.w, u.w, act, limit);
    if constexpr (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(out + 4 * i) = make_float4(r0, r1, r2, r3);
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&lo);
        raw.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + 4 * i) = raw;
    }
}

constexpr int kNrsWarps = 4;
constexpr int kNrsMaxHead = 256;

// A warp per head (query heads first, then key heads), a lane per pair of dimensions: both members of a rotation
// pair are the lane's own, the head's sum of squares is one warp reduction, nothing goes through shared memory but
// the token's sines and cosines, which all heads of the block share. Many rows: a block per token; few rows (decoding):
// a block per token and four heads. Head sizes up to 256 (four pairs a lane), even.
constexpr int kNrsPairs = kNrsMaxHead / 64;

template <typename T>
__global__ void __launch_bounds__(kNrsWarps * 32)
norm_rope_store_kernel(const float* __restrict__ in, int ld, int q_off, int k_off, int v_off,
                       const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                       const float* __restrict__ freq, int rot_half, int interleaved,
                       const int* __restrict__ positions, const int* __restrict__ row_req,
                       const int* __restrict__ block_tables, int table_stride,
                       T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                       int H, int Hkv, int hd, int vd, int page_size, int write_kv, int wide) {
    pdl_prologue();
    __shared__ float s_cos[kNrsMaxHead / 2], s_sin[kNrsMaxHead / 2];
    __shared__ float s_wide[2][kNrsWarps];
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int half = freq ? rot_half : 0;
    for (int i = threadIdx.x; i < half; i += kNrsWarps * 32) sincosf(static_cast<float>(pos) * freq[i], &s_sin[i], &s_cos[i]);
    const float* row = in + static_cast<size_t>(t) * ld;
    // wide: one unit-RMS norm over all query heads' values together (and one over all key heads'), the weights
    // [H * hd] and [Hkv * hd]; every block of the token takes the two sums over the whole row in the same order
    if (wide) {
        float sq = 0.f, sk = 0.f;
        if (q_norm) for (int i = threadIdx.x; i < H * hd; i += kNrsWarps * 32) sq = fmaf(row[q_off + i], row[q_off + i], sq);
        if (k_norm) for (int i = threadIdx.x; i < Hkv * hd; i += kNrsWarps * 32) sk = fmaf(row[k_off + i], row[k_off + i], sk);
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { s_wide[0][warp] = sq; s_wide[1][warp] = sk; }
    }
    __syncthreads();
    float wide_scale[2] = {1.f, 1.f};
    if (wide) {
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int w = 0; w < kNrsWarps; ++w) { sq += s_wide[0][w]; sk += s_wide[1][w]; }
        wide_scale[0] = 1.0f / sqrtf(sq / static_cast<float>(H * hd) + eps);
        wide_scale[1] = 1.0f / sqrtf(sk / static_cast<float>(Hkv * hd) + eps);
    }
    size_t kv_base = 0, v_base = 0;       // in rows: a value row has vd values, a key row hd
    if (write_kv) {
        const int page = block_tables[static_cast<size_t>(row_req[t]) * table_stride + pos / page_size];
        kv_base = (static_cast<size_t>(page) * Hkv * page_size + (pos % page_size)) * hd;
        v_base = (static_cast<size_t>(page) * Hkv * page_size + (pos % page_size)) * vd;
    }
    const int n_heads = H + (write_kv ? Hkv : 0);
    const int n_pairs = hd / 2;
    for (int head = blockIdx.y * kNrsWarps + warp; head < n_heads; head += kNrsWarps * gridDim.y) {
        const bool is_q = head < H;
        const float* src = row + (is_q ? q_off + head * hd : k_off + (head - H) * hd);
        const float* nw = is_q ? q_norm : k_norm;
        if (nw && wide) nw += (is_q ? head : head - H) * hd;
        float va[kNrsPairs], vb[kNrsPairs];
        int ia[kNrsPairs], ib[kNrsPairs];
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < kNrsPairs; ++u) {
            const int pr = lane + 32 * u;
            // pair pr: a rotation pair while pr < half, else two neighbouring dimensions behind the rotated ones
            if (interleaved || pr >= half) {
                const int base = interleaved ? 2 * pr : 2 * half + 2 * (pr - half);
                ia[u] = base; ib[u] = base + 1;
            } else {
                ia[u] = pr; ib[u] = pr + half;
            }
            const bool in_head = pr < n_pairs;
            va[u] = in_head ? src[ia[u]] : 0.f;
            vb[u] = in_head ? src[ib[u]] : 0.f;
            ss = fmaf(va[u], va[u], ss);
            ss = fmaf(vb[u], vb[u], ss);
        }
        T* dst = is_q ? q_out + (static_cast<size_t>(t) * H + head) * hd
                      : k_cache + kv_base + static_cast<size_t>(head - H) * page_size * hd;
        if (!is_q) {
            // the values: copied from their columns as they are (the keys themselves where the design says so)
            const float* vsrc = row + v_off + (head - H) * vd;
            T* vdst = v_cache + v_base + static_cast<size_t>(head - H) * page_size * vd;
            for (int d = lane; d < vd; d += 32) vdst[d] = from_float<T>(vsrc[d]);
        }
        if (nw) {
            ss = warp_sum(ss);
            const float scale = wide ? wide_scale[is_q ? 0 : 1] : 1.0f / sqrtf(ss / static_cast<float>(hd) + eps);
#pragma unroll
            for (int u = 0; u < kNrsPairs; ++u) {
                if (lane + 32 * u < n_pairs) {
                    va[u] = nw[ia[u]] * (scale * va[u]);
                    vb[u] = nw[ib[u]] * (scale * vb[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kNrsPairs; ++u) {
            const int pr = lane + 32 * u;
            if (pr >= n_pairs) continue;
            float a = va[u], b = vb[u];
            if (pr < half) {
                const float sn = s_sin[pr], cs = s_cos[pr];
                const float ra = a * cs - b * sn, rb = b * cs + a * sn;
                a = ra; b = rb;
            }
            dst[ia[u]] = from_float<T>(a);
            dst[ib[u]] = from_float<T>(b);
        }
    }
}

template <typename TOut>
__global__ void __launch_bounds__(256)
add_normed_kernel(float* __restrict__ y, const float* __restrict__ weight, float* __restrict__ x, TOut* __restrict__ xn_out,
                  int D, float eps, int clear_y) {
    pdl_prologue();
    __shared__ float warp_part[8];
    const size_t row = static_cast<size_t>(blockIdx.x) * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += 256) ss = fmaf(y[row + d], y[row + d], ss);
    const float total = block_sum_256(ss, warp_part);
    const float scale = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
    for (int d = threadIdx.x; d < D; d += 256) {
        const float v = x[row + d] + weight[d] * (scale * y[row + d]);
        x[row + d] = v;
        if (xn_out) xn_out[row + d] = from_float<TOut>(v);
        if (clear_y) y[row + d] = 0.f;
    }
}

// One block per token. The two latents are normed by the block (sums in the order of block_sum_256); the rotated part
// is a pair per thread.
template <typename T>
__global__ void __launch_bounds__(256)
latent_store_kernel(const float* __restrict__ in, int ld, int q_off, int q_rank, const float* __restrict__ q_weight,
                    T* __restrict__ q_latent, int c_off, int rank, const float* __restrict__ c_weight, int r_off, int rot,
                    const float* __restrict__ freq, float amplitude, float eps, const int* __restrict__ positions,
                    const int* __restrict__ row_req, const int* __restrict__ block_tables, int table_stride,
                    T* __restrict__ cache, int page_size, int write_cache) {
    pdl_prologue();
    __shared__ float warp_part[8];
    const int t = blockIdx.x;
    const float* row = in + static_cast<size_t>(t) * ld;
    if (q_latent) {
        float ss = 0.f;
        for (int d = threadIdx.x; d < q_rank; d += 256) ss = fmaf(row[q_off + d], row[q_off + d], ss);
        const float scale = 1.0f / sqrtf(block_sum_256(ss, warp_part) / static_cast<float>(q_rank) + eps);
        for (int d = threadIdx.x; d < q_rank; d += 256)
            q_latent[static_cast<size_t>(t) * q_rank + d] = from_float<T>(q_weight[d] * (scale * row[q_off + d]));
    }
    if (!write_cache) return;
    const int pos = positions[t];
    const int page = block_tables[static_cast<size_t>(row_req[t]) * table_stride + pos / page_size];
    T* dst = cache + (static_cast<size_t>(page) * page_size + (pos % page_size)) * (rank + rot);
    float ss = 0.f;
    for (int d = threadIdx.x; d < rank; d += 256) ss = fmaf(row[c_off + d], row[c_off + d], ss);
    const float scale = 1.0f / sqrtf(block_sum_256(ss, warp_part) / static_cast<float>(rank) + eps);
    for (int d = threadIdx.x; d < rank; d += 256) dst[d] = from_float<T>(c_weight[d] * (scale * row[c_off + d]));
    for (int pr = threadIdx.x; pr < rot / 2; pr += 256) {
        float sn, cs;
        sincosf(static_cast<float>(pos) * freq[pr], &sn, &cs);
        sn *= amplitude; cs *= amplitude;
        const float u = row[r_off + 2 * pr], v = row[r_off + 2 * pr + 1];
        dst[rank + 2 * pr] = from_float<T>(u * cs - v * sn);
        dst[rank + 2 * pr + 1] = from_float<T>(v * cs + u * sn);
    }
}

}  // namespace gi

using namespace gi;

static int gi_scale_cast_impl(const float* x, float* acc, void* xn, int xn_dtype, float alpha, long long total, void* stream) {
    if (total == 0) return 0;
    GI_REQUIRE(total > 0, "scale_cast: the size must be positive");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 148 * 16));
    if (xn_dtype == kBF16)
        launch_kernel((scale_cast_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, st, x, acc, static_cast<__nv_bfloat16*>(xn), alpha, static_cast<size_t>(total));
    else
        launch_kernel((scale_cast_kernel<float>), dim3(blocks), dim3(256), 0, st, x, acc, static_cast<float*>(xn), alpha, static_cast<size_t>(total));
    return check_launch("scale_cast");
}

static int gi_residual_norm_impl(const float* acc_in, const float* weight, float* x_out, float* acc_out, void* xn_out,
                                 int xn_dtype, int rows, int D, float eps, float alpha, void* stream) {
    if (rows == 0) return 0;
    GI_REQUIRE(rows > 0 && D > 0, "residual_norm: sizes must be positive (rows=%d, D=%d)", rows, D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (xn_dtype == kBF16)
        launch_kernel((residual_norm_kernel<__nv_bfloat16>), dim3(rows), dim3(256), 0, st, acc_in, weight, x_out, acc_out,
                      static_cast<__nv_bfloat16*>(xn_out), D, eps, alpha);
    else
        launch_kernel((residual_norm_kernel<float>), dim3(rows), dim3(256), 0, st, acc_in, weight, x_out, acc_out,
                      static_cast<float*>(xn_out), D, eps, alpha);
    return check_launch("residual_norm");
}

static int gi_gated_act_impl(const float* gate_up, const float* bias, void* out, int out_dtype, int T, int I, int act, float limit, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && I > 0, "gated_act: sizes must be positive (T=%d, I=%d)", T, I);
    GI_REQUIRE(act >= 0 && act < kActCount, "gated_act: unknown activation code %d", act);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t total = static_cast<size_t>(T) * I;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    if (I % 4 == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(bias) % 16 == 0 && (out_dtype == kBF16 || out_dtype == kF32)) {
        const unsigned blocks4 = static_cast<unsigned>((total / 4 + 255) / 256);
        if (out_dtype == kBF16)
            launch_kernel((gated_act4_kernel<__nv_bfloat16>), dim3(blocks4), dim3(256), 0, st, gate_up, bias, static_cast<__nv_bfloat16*>(out), I / 4, total / 4, act, limit);
        else
            launch_kernel((gated_act4_kernel<float>), dim3(blocks4), dim3(256), 0, st, gate_up, bias, static_cast<float*>(out), I / 4, total / 4, act, limit);
        return check_launch("gated_act");
    }
    if (out_dtype == kBF16)
        launch_kernel((gated_act_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, st, gate_up, bias, static_cast<__nv_bfloat16*>(out), I, total, act, limit);
    else if (out_dtype == kF32)
        launch_kernel((gated_act_kernel<float>), dim3(blocks), dim3(256), 0, st, gate_up, bias, static_cast<float*>(out), I, total, act, limit);
    else
        GI_REQUIRE(false, "gated_act: unsupported output dtype code %d", out_dtype);
    return check_launch("gated_act");
}

static int gi_norm_rope_store_impl(const float* in, int ld, int q_off, int k_off, int v_off, const float* q_norm,
                                   const float* k_norm, float eps, const float* freq, int rot_half, int interleaved,
                                   const int* positions, const int* row_req, const int* block_tables, int table_stride,
                                   void* q_out, void* k_cache, void* v_cache, int dtype, int T, int H, int Hkv, int hd,
                                   int vd, int page_size, int write_kv, int wide, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && H > 0 && Hkv > 0 && hd > 0 && page_size > 0, "norm_rope_store: sizes must be positive");
    GI_REQUIRE(hd <= kNrsMaxHead && hd % 2 == 0, "norm_rope_store: head size %d is odd or exceeds %d", hd, kNrsMaxHead);
    GI_REQUIRE(2 * rot_half <= hd, "norm_rope_store: rotary size %d exceeds the head size %d", 2 * rot_half, hd);
    GI_REQUIRE(vd > 0, "norm_rope_store: the value size must be positive");
    GI_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + H * hd <= ld && k_off + Hkv * hd <= ld && v_off + Hkv * vd <= ld,
               "norm_rope_store: the columns of queries, keys or values lie outside the input row of %d", ld);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    GI_REQUIRE(T <= 2147483647, "norm_rope_store: too many rows");
    // few rows (decoding): the heads of a token are spread over blocks; many rows: a block per token
    const unsigned head_blocks = T >= 256 ? 1u : static_cast<unsigned>(std::min((H + Hkv + kNrsWarps - 1) / kNrsWarps, 65535));
    if (dtype == kF32)
        launch_kernel((norm_rope_store_kernel<float>), dim3(T, head_blocks), dim3(kNrsWarps * 32), 0, st, in, ld, q_off, k_off, v_off, q_norm,
                      k_norm, eps, freq, rot_half, interleaved, positions, row_req, block_tables, table_stride,
                      static_cast<float*>(q_out), static_cast<float*>(k_cache), static_cast<float*>(v_cache), H, Hkv, hd,
                      vd, page_size, write_kv, wide);
    else if (dtype == kBF16)
        launch_kernel((norm_rope_store_kernel<__nv_bfloat16>), dim3(T, head_blocks), dim3(kNrsWarps * 32), 0, st, in, ld, q_off, k_off, v_off,
                      q_norm, k_norm, eps, freq, rot_half, interleaved, positions, row_req, block_tables, table_stride,
                      static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                      static_cast<__nv_bfloat16*>(v_cache), H, Hkv, hd, vd, page_size, write_kv, wide);
    else
        GI_REQUIRE(false, "norm_rope_store: unsupported dtype code %d", dtype);
    return check_launch("norm_rope_store");
}

extern "C" int gi_scale_cast(const float* x, float* acc, void* xn, int xn_dtype, float alpha, long long total, void* stream) {
    return gi::dispatch(gi_scale_cast_impl, x, acc, xn, xn_dtype, alpha, total, stream);
}

extern "C" int gi_residual_norm(const float* acc_in, const float* weight, float* x_out, float* acc_out, void* xn_out, int xn_dtype, int rows, int D, float eps, float alpha, void* stream) {
    return gi::dispatch(gi_residual_norm_impl, acc_in, weight, x_out, acc_out, xn_out, xn_dtype, rows, D, eps, alpha, stream);
}

extern "C" int gi_gated_act(const float* gate_up, const float* bias, void* out, int out_dtype, int T, int I, int act, float limit, void* stream) {
    return gi::dispatch(gi_gated_act_impl, gate_up, bias, out, out_dtype, T, I, act, limit, stream);
}

extern "C" int gi_norm_rope_store(const float* in, int ld, int q_off, int k_off, int v_off, const float* q_norm, const float* k_norm, float eps, const float* freq, int rot_half, int interleaved, const int* positions, const int* row_req, const int* block_tables, int table_stride, void* q_out, void* k_cache, void* v_cache, int dtype, int T, int H, int Hkv, int hd, int vd, int page_size, int write_kv, int wide, void* stream) {
    return gi::dispatch(gi_norm_rope_store_impl, in, ld, q_off, k_off, v_off, q_norm, k_norm, eps, freq, rot_half, interleaved, positions, row_req, block_tables, table_stride, q_out, k_cache, v_cache, dtype, T, H, Hkv, hd, vd, page_size, write_kv, wide, stream);
}

static int gi_add_normed_impl(float* y, const float* weight, float* x, void* xn_out, int xn_dtype, int rows, int D, float eps,
                              int clear_y, void* stream) {
    if (rows == 0) return 0;
    GI_REQUIRE(rows > 0 && D > 0, "add_normed: sizes must be positive (rows=%d, D=%d)", rows, D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (xn_dtype == kBF16)
        launch_kernel((add_normed_kernel<__nv_bfloat16>), dim3(rows), dim3(256), 0, st, y, weight, x, static_cast<__nv_bfloat16*>(xn_out), D, eps, clear_y);
    else
        launch_kernel((add_normed_kernel<float>), dim3(rows), dim3(256), 0, st, y, weight, x, static_cast<float*>(xn_out), D, eps, clear_y);
    return check_launch("add_normed");
}

static int gi_latent_store_impl(const float* in, int ld, int q_off, int q_rank, const float* q_weight, void* q_latent, int c_off,
                                int rank, const float* c_weight, int r_off, int rot, const float* freq, float amplitude, float eps,
                                const int* positions, const int* row_req, const int* block_tables, int table_stride, void* cache,
                                int dtype, int T, int page_size, int write_cache, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && page_size > 0, "latent_store: sizes must be positive and the rotated part even");
    GI_REQUIRE(q_latent == nullptr || (q_rank > 0 && q_weight && q_off >= 0 && q_off + q_rank <= ld), "latent_store: the query latent lies outside the row");
    GI_REQUIRE(c_off >= 0 && c_off + rank <= ld && r_off >= 0 && r_off + rot <= ld, "latent_store: the key/value latent lies outside the row of %d", ld);
    GI_REQUIRE(rot == 0 || freq, "latent_store: the rotated part needs frequencies");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == kF32)
        launch_kernel((latent_store_kernel<float>), dim3(T), dim3(256), 0, st, in, ld, q_off, q_rank, q_weight, static_cast<float*>(q_latent),
                      c_off, rank, c_weight, r_off, rot, freq, amplitude, eps, positions, row_req, block_tables, table_stride,
                      static_cast<float*>(cache), page_size, write_cache);
    else if (dtype == kBF16)
        launch_kernel((latent_store_kernel<__nv_bfloat16>), dim3(T), dim3(256), 0, st, in, ld, q_off, q_rank, q_weight,
                      static_cast<__nv_bfloat16*>(q_latent), c_off, rank, c_weight, r_off, rot, freq, amplitude, eps, positions, row_req,
                      block_tables, table_stride, static_cast<__nv_bfloat16*>(cache), page_size, write_cache);
    else
        GI_REQUIRE(false, "latent_store: unsupported dtype code %d", dtype);
    return check_launch("latent_store");
}

extern "C" int gi_add_normed(float* y, const float* weight, float* x, void* xn_out, int xn_dtype, int rows, int D, float eps, int clear_y, void* stream) {
    return gi::dispatch(gi_add_normed_impl, y, weight, x, xn_out, xn_dtype, rows, D, eps, clear_y, stream);
}

extern "C" int gi_latent_store(const float* in, int ld, int q_off, int q_rank, const float* q_weight, void* q_latent, int c_off, int rank, const float* c_weight, int r_off, int rot, const float* freq, float amplitude, float eps, const int* positions, const int* row_req, const int* block_tables, int table_stride, void* cache, int dtype, int T, int page_size, int write_cache, void* stream) {
    return gi::dispatch(gi_latent_store_impl, in, ld, q_off, q_rank, q_weight, q_latent, c_off, rank, c_weight, r_off, rot, freq, amplitude, eps, positions, row_req, block_tables, table_stride, cache, dtype, T, page_size, write_cache, stream);
}
