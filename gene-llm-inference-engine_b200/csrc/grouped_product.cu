// Matrix products whose weight matrix depends on the row: one matrix per head, or one per expert.
//
//   grouped_product   out[row, g-th slice] (=) W[g] a[row, g-th slice]  for tiles of 16 rows that share a group g
//     heads    every row (token) runs through every group (head) h: a's columns a_off + h * a_gs .. + K,
//              W[h] = w + h * w_gs [N, K], out's columns o_off + h * o_gs .. + N; optionally ``tail`` more
//              columns behind a head's K inputs are rotated by the row's position and copied behind its N outputs
//              (queries of an attention over a shared latent: the plain part goes through the head's key matrix,
//              the rotated part stays); optionally every output is multiplied by the sigmoid of a gate value of its own
//              (32-bit, in a row of the token: the heads' outputs of a gated attention)
//     experts  rows are (token, choice) pairs sorted by expert: tile i belongs to expert tile_group[i], its rows are
//              sorted_rows[16 i ..] (-1: none); the input row is pair / a_div, the output row the pair;
//              gated: out = act(W_gate a) * (W_up a) with W[g] = [gate rows; up rows]
//   route             per token: z = W_r x in 32-bit, s = sigmoid(z), the ``top`` experts by s + correction, weights s
//   route_align       buckets the pairs by expert into tiles of 16 rows (padding with -1), one block; for many rows
//                     into tiles of 128, the token tiles of the tensor-core product that takes a matrix per tile
//   gather_rows       a[r] = x[sorted_rows[r] / top] (zeros for padding): the rows in the tiles' order
//   route_combine     y[t] += sum_k weight[t, k] * part[row of pair t * top + k] in the order of k
//
// Products run on the CUDA cores with 32-bit fused multiply-adds: the true 32-bit path, products of few rows (decoding,
// where the weights stream once), the heads' matrices, and the bfloat16 path's fallback. Three forms: tiles of 16 x 64
// outputs, tiles of 64 x 64 (many rows through the heads' matrices) and the few-row form further down. In the tiled forms
// an output element is one chain of multiply-adds in the order of k over its own row, whichever tile the row landed in;
// in the few-row form it is the sum of a warp's lanes' chains by a fixed tree. (Many rows through the experts' matrices
// in bfloat16 run on the tensor cores: gi_gemm_tc_grouped.)
#include "common.cuh"

namespace gi {

constexpr int kGpTM = 16, kGpTN = 64, kGpTK = 32;

struct GroupedArgs {
    const void* a; long long lda; int a_off; int a_gs; int a_div;
    const void* w; long long w_gs; int ldw; long long up_off;     // W[g] = w + g * w_gs, rows of ldw; the up rows start at up_off
    void* out; int out_is_f32; long long ldo; int o_off; int o_gs;
    int N, K, rows, groups;
    const int* tile_group; const int* sorted_rows; const int* n_tiles;   // experts form (else null)
    int act; float act_limit;                                     // gated: a GateAct code and its limit
    // rotated tail (heads form)
    int tail; const float* freq; float amplitude; const int* positions;
    // output gate (heads form): out *= sigmoid(gate[row, gate_off + h * N + n]), 32-bit (else null)
    const float* gate; long long ldg; int gate_off;
};

// The element-wise sigmoid gate of the heads form, on output n of head g of row r.
__device__ __forceinline__ float gp_gated(const GroupedArgs& p, float v, int r, int g, int n) {
    if (p.gate == nullptr) return v;
    const float z = p.gate[static_cast<size_t>(r) * p.ldg + p.gate_off + static_cast<size_t>(g) * p.N + n];
    return v * (1.0f / (1.0f + expf(-z)));
}

template <typename TA, typename TW, bool GATED>
__global__ void __launch_bounds__(128)
grouped_product_kernel(const GroupedArgs p) {
    pdl_prologue();
    constexpr int U = GATED ? 1 : 0;
    __shared__ float s_a[kGpTK][kGpTM + 1];
    __shared__ __align__(16) float s_w[U + 1][kGpTK][kGpTN + 4];
    __shared__ int s_row[kGpTM];

    const int tid = threadIdx.x;
    int g, row0 = 0;
    if (p.tile_group) {
        if (static_cast<int>(blockIdx.x) >= *p.n_tiles) return;
        g = p.tile_group[blockIdx.x];
        if (tid < kGpTM) s_row[tid] = p.sorted_rows[blockIdx.x * kGpTM + tid];
    } else {
        g = blockIdx.x % p.groups;
        row0 = (blockIdx.x / p.groups) * kGpTM;
        if (tid < kGpTM) s_row[tid] = row0 + tid < p.rows ? row0 + tid : -1;
    }
    __syncthreads();
    const int n0 = blockIdx.y * kGpTN;
    const TA* A = static_cast<const TA*>(p.a);
    const TW* W = static_cast<const TW*>(p.w) + static_cast<size_t>(g) * p.w_gs;

    // rotated tail: only the blocks of the first tile of outputs do it
    if (p.tail > 0 && blockIdx.y == 0) {
        for (int i = tid; i < kGpTM * (p.tail / 2); i += 128) {
            const int m = i / (p.tail / 2), pr = i % (p.tail / 2);
            const int r = s_row[m];
            if (r < 0) continue;
            const TA* src = A + static_cast<size_t>(r) * p.lda + p.a_off + static_cast<size_t>(g) * p.a_gs + p.K + 2 * pr;
            float sn, cs;
            sincosf(static_cast<float>(p.positions[r]) * p.freq[pr], &sn, &cs);
            sn *= p.amplitude; cs *= p.amplitude;
            const float u = to_float(src[0]), v = to_float(src[1]);
            const size_t o = static_cast<size_t>(r) * p.ldo + p.o_off + static_cast<size_t>(g) * p.o_gs + p.N + 2 * pr;
            const float ru = u * cs - v * sn, rv = v * cs + u * sn;
            if (p.out_is_f32) { static_cast<float*>(p.out)[o] = ru; static_cast<float*>(p.out)[o + 1] = rv; }
            else { static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(ru); static_cast<__nv_bfloat16*>(p.out)[o + 1] = __float2bfloat16_rn(rv); }
        }
    }

    const int tm = (tid >> 4) * 2, tn = (tid & 15) * 4;
    float acc[2][4] = {}, acc_up[U + 1][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += kGpTK) {
        // rows of a: 16 x 32 values
        for (int i = tid; i < kGpTM * kGpTK; i += 128) {
            const int m = i / kGpTK, k = i % kGpTK;
            const int r = s_row[m];
            float v = 0.f;
            if (r >= 0 && k0 + k < p.K)
                v = to_float(A[static_cast<size_t>(r / p.a_div) * p.lda + p.a_off + static_cast<size_t>(g) * p.a_gs + k0 + k]);
            s_a[k][m] = v;
        }
        // rows of W: 64 x 32 values (and the up rows)
        for (int i = tid; i < kGpTN * kGpTK; i += 128) {
            const int n = i / kGpTK, k = i % kGpTK;
            const bool in = n0 + n < p.N && k0 + k < p.K;
            const size_t off = static_cast<size_t>(n0 + n) * p.ldw + k0 + k;
            s_w[0][k][n] = in ? to_float(W[off]) : 0.f;
            if (GATED) s_w[U][k][n] = in ? to_float(W[p.up_off + off]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < kGpTK; ++k) {
            const float a0 = s_a[k][tm], a1 = s_a[k][tm + 1];
            const float4 w4 = *reinterpret_cast<const float4*>(&s_w[0][k][tn]);
            acc[0][0] = fmaf(a0, w4.x, acc[0][0]); acc[0][1] = fmaf(a0, w4.y, acc[0][1]);
            acc[0][2] = fmaf(a0, w4.z, acc[0][2]); acc[0][3] = fmaf(a0, w4.w, acc[0][3]);
            acc[1][0] = fmaf(a1, w4.x, acc[1][0]); acc[1][1] = fmaf(a1, w4.y, acc[1][1]);
            acc[1][2] = fmaf(a1, w4.z, acc[1][2]); acc[1][3] = fmaf(a1, w4.w, acc[1][3]);
            if (GATED) {
                const float4 u4 = *reinterpret_cast<const float4*>(&s_w[U][k][tn]);
                acc_up[0][0] = fmaf(a0, u4.x, acc_up[0][0]); acc_up[0][1] = fmaf(a0, u4.y, acc_up[0][1]);
                acc_up[0][2] = fmaf(a0, u4.z, acc_up[0][2]); acc_up[0][3] = fmaf(a0, u4.w, acc_up[0][3]);
                acc_up[U][0] = fmaf(a1, u4.x, acc_up[U][0]); acc_up[U][1] = fmaf(a1, u4.y, acc_up[U][1]);
                acc_up[U][2] = fmaf(a1, u4.z, acc_up[U][2]); acc_up[U][3] = fmaf(a1, u4.w, acc_up[U][3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = s_row[tm + i];
        if (r < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n >= p.N) continue;
            float v = acc[i][j];
            if (GATED) v = gated_value(v, acc_up[U * i][j], p.act, p.act_limit);
            v = gp_gated(p, v, r, g, n);
            const size_t o = static_cast<size_t>(r) * p.ldo + p.o_off + static_cast<size_t>(g) * p.o_gs + n;
            if (p.out_is_f32) static_cast<float*>(p.out)[o] = v;
            else static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
        }
    }
}

// The same products for few rows (decoding): the weights are what takes the time, so a warp streams whole rows of a
// group's matrix with 16-byte loads, four rows after one another, and multiplies each with every row of the tile (at most
// 16, read through the cache); a block of eight warps covers 32 output rows, so a matrix of a few thousand rows is spread
// over more than a hundred blocks per tile. An output element is the sum of its lanes' partial sums (lane l takes the
// pieces l, l + 32, ...), added by a fixed xor tree: it depends on its own row only.
constexpr int kGrRows = 32;           // output rows per block
constexpr int kGrFew = 4;             // rows of a tile that are multiplied with a piece of the weights while it is in registers

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
};

// PIECE: values per step of a lane = the weights' 16 bytes (8 bfloat16 or 4 floats); the inputs are read in as many.
template <typename TA, typename TW, bool GATED>
__global__ void __launch_bounds__(256)
grouped_rows_kernel(const GroupedArgs p) {
    pdl_prologue();
    constexpr int PIECE = Vec16<TW>::N;
    __shared__ int s_row[kGpTM];
    __shared__ int s_count;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int g;
    if (p.tile_group) {
        if (static_cast<int>(blockIdx.x) >= *p.n_tiles) return;
        g = p.tile_group[blockIdx.x];
    } else {
        g = blockIdx.x % p.groups;
    }
    if (tid == 0) {             // the tile's rows, the empty places left out
        int n = 0;
        for (int i = 0; i < kGpTM; ++i) {
            int r;
            if (p.tile_group) r = p.sorted_rows[blockIdx.x * kGpTM + i];
            else { r = (blockIdx.x / p.groups) * kGpTM + i; if (r >= p.rows) r = -1; }
            if (r >= 0) s_row[n++] = r;
        }
        s_count = n;
    }
    __syncthreads();
    const int m_count = s_count;
    const TA* A = static_cast<const TA*>(p.a) + p.a_off + static_cast<size_t>(g) * p.a_gs;
    const TW* W = static_cast<const TW*>(p.w) + static_cast<size_t>(g) * p.w_gs;
    const int pieces = p.K / PIECE;
    // The warp's four weight rows are streamed together, eight 16-byte loads of a lane in flight, and every input piece is
    // read once for the four. The tile's rows are taken four at a time (a tile of a decode step seldom has more); a
    // second group of four streams the same weight rows again, from the L2 cache.
    const int n_first = blockIdx.y * kGrRows + warp * 4;
    if (n_first >= p.N) return;
    const TW* wrow[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) wrow[r] = W + static_cast<size_t>(min(n_first + r, p.N - 1)) * p.ldw;
    for (int m0 = 0; m0 < m_count; m0 += kGrFew) {
        const int m_here = min(kGrFew, m_count - m0);
        float acc[4][kGrFew], acc_up[GATED ? 4 : 1][kGrFew];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < kGrFew; ++i) { acc[r][i] = 0.f; if (GATED) acc_up[GATED ? r : 0][i] = 0.f; }
        }
        // the output gate's values of the warp's 4 x kGrFew outputs, a lane each, asked for before the weights stream
        float gate_z = 0.f;
        if (p.gate != nullptr && lane < 4 * kGrFew) {
            const int gr = lane / kGrFew, gi_ = lane % kGrFew;
            if (gi_ < m_here && n_first + gr < p.N)
                gate_z = p.gate[static_cast<size_t>(s_row[m0 + gi_]) * p.ldg + p.gate_off + static_cast<size_t>(g) * p.N + n_first + gr];
        }
        for (int c = lane; c < pieces; c += 32) {
            float wv[4][8], uv[GATED ? 4 : 1][8];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                Vec16<TW>::load(wrow[r] + c * PIECE, wv[r]);
                if (GATED) Vec16<TW>::load(wrow[r] + p.up_off + c * PIECE, uv[GATED ? r : 0]);
            }
#pragma unroll
            for (int i = 0; i < kGrFew; ++i) {
                if (i < m_here) {
                    const TA* arow = A + static_cast<size_t>(s_row[m0 + i] / p.a_div) * p.lda + c * PIECE;
                    float av[8];
                    if (sizeof(TA) == 4 && PIECE == 8) {          // 32-bit inputs against bfloat16 weights: two loads
                        float lo4[8], hi4[8];
                        Vec16<float>::load(reinterpret_cast<const float*>(arow), lo4);
                        Vec16<float>::load(reinterpret_cast<const float*>(arow) + 4, hi4);
#pragma unroll
                        for (int j = 0; j < 4; ++j) { av[j] = lo4[j]; av[4 + j] = hi4[j]; }
                    } else {
                        Vec16<TA>::load(arow, av);
                    }
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
#pragma unroll
                        for (int j = 0; j < PIECE; ++j) {
                            acc[r][i] = fmaf(av[j], wv[r][j], acc[r][i]);
                            if (GATED) acc_up[GATED ? r : 0][i] = fmaf(av[j], uv[GATED ? r : 0][j], acc_up[GATED ? r : 0][i]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < kGrFew; ++i) {
                if (i < m_here && n_first + r < p.N) {
                    float v = warp_sum(acc[r][i]);
                    if (GATED) v = gated_value(v, warp_sum(acc_up[GATED ? r : 0][i]), p.act, p.act_limit);
                    if (p.gate != nullptr) v *= 1.0f / (1.0f + expf(-__shfl_sync(0xffffffffu, gate_z, r * kGrFew + i)));
                    if (lane == 0) {
                        const size_t o = static_cast<size_t>(s_row[m0 + i]) * p.ldo + p.o_off + static_cast<size_t>(g) * p.o_gs + n_first + r;
                        if (p.out_is_f32) static_cast<float*>(p.out)[o] = v;
                        else static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
    }
}

// The heads form for many rows (prompt portions): tiles of 64 rows x 64 outputs, a thread 4 x 4 of them, so that two
// 16-byte reads of shared memory feed sixteen multiply-adds. Inputs 32-bit or bfloat16, weights likewise; rows of four
// values must be aligned (the caller checks). An output element is one chain of multiply-adds in the order of k.
constexpr int kG64 = 64, kG64K = 16;

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
head_product64_kernel(const GroupedArgs p) {
    pdl_prologue();
    __shared__ __align__(16) float s_a[kG64K][kG64 + 4];
    __shared__ __align__(16) float s_w[kG64K][kG64 + 4];
    const int tid = threadIdx.x;
    const int g = blockIdx.x % p.groups;
    const int row0 = (blockIdx.x / p.groups) * kG64;
    const int n0 = blockIdx.y * kG64;
    const TA* A = static_cast<const TA*>(p.a) + p.a_off + static_cast<size_t>(g) * p.a_gs;
    const TW* W = static_cast<const TW*>(p.w) + static_cast<size_t>(g) * p.w_gs;

    if (p.tail > 0 && blockIdx.y == 0) {            // the rotated tail, by the blocks of the first tile of outputs
        for (int i = tid; i < kG64 * (p.tail / 2); i += 256) {
            const int m = i / (p.tail / 2), pr = i % (p.tail / 2);
            const int r = row0 + m;
            if (r >= p.rows) continue;
            const TA* src = A + static_cast<size_t>(r) * p.lda + p.K + 2 * pr;
            float sn, cs;
            sincosf(static_cast<float>(p.positions[r]) * p.freq[pr], &sn, &cs);
            sn *= p.amplitude; cs *= p.amplitude;
            const float u = to_float(src[0]), v = to_float(src[1]);
            const size_t o = static_cast<size_t>(r) * p.ldo + p.o_off + static_cast<size_t>(g) * p.o_gs + p.N + 2 * pr;
            const float ru = u * cs - v * sn, rv = v * cs + u * sn;
            if (p.out_is_f32) { static_cast<float*>(p.out)[o] = ru; static_cast<float*>(p.out)[o + 1] = rv; }
            else { static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(ru); static_cast<__nv_bfloat16*>(p.out)[o + 1] = __float2bfloat16_rn(rv); }
        }
    }

    const int lr = tid >> 2, lk = (tid & 3) * 4;             // what this thread brings in: row (or output) lr, values lk..lk+3
    const int ty = (tid >> 4) * 4, tx = (tid & 15) * 4;      // its 4 x 4 outputs
    float acc[4][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += kG64K) {
        float4 av = make_float4(0.f, 0.f, 0.f, 0.f), wv = av;
        if (row0 + lr < p.rows && k0 + lk < p.K) av = load4<TA>(A + static_cast<size_t>(row0 + lr) * p.lda + k0 + lk);
        if (n0 + lr < p.N && k0 + lk < p.K) wv = load4<TW>(W + static_cast<size_t>(n0 + lr) * p.ldw + k0 + lk);
        __syncthreads();                                      // the tile before is done with
        s_a[lk][lr] = av.x; s_a[lk + 1][lr] = av.y; s_a[lk + 2][lr] = av.z; s_a[lk + 3][lr] = av.w;
        s_w[lk][lr] = wv.x; s_w[lk + 1][lr] = wv.y; s_w[lk + 2][lr] = wv.z; s_w[lk + 3][lr] = wv.w;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kG64K; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&s_a[k][ty]);
            const float4 w4 = *reinterpret_cast<const float4*>(&s_w[k][tx]);
            const float ar[4] = {a4.x, a4.y, a4.z, a4.w}, wr[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty + i;
        if (r >= p.rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + j;
            if (n >= p.N) continue;
            const size_t o = static_cast<size_t>(r) * p.ldo + p.o_off + static_cast<size_t>(g) * p.o_gs + n;
            const float v = gp_gated(p, acc[i][j], r, g, n);
            if (p.out_is_f32) static_cast<float*>(p.out)[o] = v;
            else static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
        }
    }
}

// ------------------------------------------------------------------------------------------------ routing
constexpr int kRouteMaxExperts = 1024;

template <typename TX>
__global__ void __launch_bounds__(128)
route_kernel(const TX* __restrict__ x, int D, const float* __restrict__ w, const float* __restrict__ correction, int E, int top,
             int* __restrict__ ids, float* __restrict__ weights) {
    pdl_prologue();
    extern __shared__ float s_x[];                 // [D]
    __shared__ float s_score[kRouteMaxExperts], s_choice[kRouteMaxExperts];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int d = threadIdx.x; d < D; d += 128) s_x[d] = to_float(x[static_cast<size_t>(t) * D + d]);
    __syncthreads();
    for (int e = warp; e < E; e += 4) {
        const float* row = w + static_cast<size_t>(e) * D;
        float z = 0.f;
        for (int d = lane; d < D; d += 32) z = fmaf(row[d], s_x[d], z);
        z = warp_sum(z);
        if (lane == 0) {
            const float s = 1.0f / (1.0f + expf(-z));
            s_score[e] = s;
            s_choice[e] = s + (correction ? correction[e] : 0.f);
        }
    }
    __syncthreads();
    if (warp != 0) return;
    // the ``top`` largest choice scores, the lowest index among equals; a chosen expert leaves the contest
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = s_choice[e];
            if (c > best) { best = c; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (lane == 0) {
            ids[static_cast<size_t>(t) * top + k] = best_e;
            weights[static_cast<size_t>(t) * top + k] = s_score[best_e];
            s_choice[best_e] = -INFINITY;
        }
        __syncwarp();
    }
}

// Experts fixed per token id: ids[t, :] = table[token of row t, :], every weight 1 / top. A token given as -(k + 1) is read
// from place k of the feedback buffer (the id a sampling kernel left on the device), as the embedding kernel reads it.
__global__ void __launch_bounds__(256)
route_table_kernel(const int* __restrict__ tokens, const int* __restrict__ feedback, const int* __restrict__ table, int vocab, int E,
                   int top, int* __restrict__ ids, float* __restrict__ weights, int n_pairs) {
    pdl_prologue();
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n_pairs) return;
    int tok = tokens[i / top];
    if (tok < 0) tok = feedback ? feedback[-tok - 1] : 0;
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    int e = table[static_cast<size_t>(tok) * top + i % top];
    e = e < 0 ? 0 : (e >= E ? E - 1 : e);                  // the table is checked when the model is built
    ids[i] = e;
    weights[i] = 1.0f / static_cast<float>(top);
}

// One block: counts per expert, then tiles of 16 rows per expert in expert order.
__global__ void __launch_bounds__(1024)
route_align_kernel(const int* __restrict__ ids, int n_pairs, int E, int* __restrict__ sorted_rows, int* __restrict__ tile_group,
                   int* __restrict__ n_tiles, int max_tiles, int tile_rows, int* __restrict__ pair_row) {
    pdl_prologue();
    __shared__ int s_count[kRouteMaxExperts], s_start[kRouteMaxExperts];
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += 1024) s_count[e] = 0;
    for (int i = tid; i < max_tiles * tile_rows; i += 1024) sorted_rows[i] = -1;
    __syncthreads();
    for (int i = tid; i < n_pairs; i += 1024) atomicAdd(&s_count[ids[i]], 1);
    __syncthreads();
    if (tid == 0) {
        int tiles = 0;
        for (int e = 0; e < E; ++e) {
            s_start[e] = tiles * tile_rows;
            const int n = (s_count[e] + tile_rows - 1) / tile_rows;
            for (int i = 0; i < n; ++i) tile_group[tiles + i] = e;
            tiles += n;
        }
        *n_tiles = tiles;
    }
    __syncthreads();
    // a pair takes the next free row of its expert (which row does not matter: an output element is computed from
    // its own row alone, in the same order of operations in every row of a tile)
    for (int i = tid; i < n_pairs; i += 1024) {
        const int row = atomicAdd(&s_start[ids[i]], 1);
        sorted_rows[row] = i;
        if (pair_row) pair_row[i] = row;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ x, int D, int a_div, const int* __restrict__ sorted_rows, const int* __restrict__ n_tiles,
                   int tile_rows, T* __restrict__ out) {
    pdl_prologue();
    const int r = blockIdx.x;
    if (r >= *n_tiles * tile_rows) return;
    const int pair = sorted_rows[r];
    T* dst = out + static_cast<size_t>(r) * D;
    if (pair < 0) {
        for (int d = threadIdx.x; d < D; d += 256) dst[d] = from_float<T>(0.f);
        return;
    }
    const T* src = x + static_cast<size_t>(pair / a_div) * D;
    if (D % 8 == 0 && sizeof(T) == 2) {
        for (int d = threadIdx.x; d < D / 8; d += 256) reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(src)[d];
    } else {
        for (int d = threadIdx.x; d < D; d += 256) dst[d] = src[d];
    }
}

__global__ void __launch_bounds__(256)
route_combine_kernel(const float* __restrict__ part, const float* __restrict__ weights, const int* __restrict__ pair_row,
                     float* __restrict__ y, int D, int top, size_t total) {
    pdl_prologue();
    const size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / D;
    const int d = static_cast<int>(i % D);
    float v = y[i];
    for (int k = 0; k < top; ++k) {
        const size_t row = pair_row ? static_cast<size_t>(pair_row[t * top + k]) : t * top + k;
        v = fmaf(weights[t * top + k], part[row * D + d], v);
    }
    y[i] = v;
}

// Whether every 16-byte load of the few-row form is aligned: pieces of the weights' rows and of the inputs' rows.
static bool rows_form_fits(const GroupedArgs& p, int a_dtype, int w_dtype) {
    const int piece = w_dtype == kBF16 ? 8 : 4;
    const size_t a_size = a_dtype == kBF16 ? 2 : 4;
    if (a_dtype == kBF16 && w_dtype == kF32) return false;
    if (p.K % piece || p.ldw % piece || p.w_gs % piece || p.up_off % piece) return false;
    if (reinterpret_cast<uintptr_t>(p.w) % 16 || reinterpret_cast<uintptr_t>(p.a) % 16) return false;
    const int a_piece = static_cast<int>(16 / a_size);
    return p.lda % a_piece == 0 && p.a_off % a_piece == 0 && p.a_gs % a_piece == 0;
}

template <bool GATED>
static int launch_grouped_rows(const GroupedArgs& p, int a_dtype, int w_dtype, unsigned tiles, cudaStream_t st) {
    dim3 grid(tiles, (p.N + kGrRows - 1) / kGrRows);
    if (a_dtype == kF32 && w_dtype == kF32) launch_kernel((grouped_rows_kernel<float, float, GATED>), grid, dim3(256), 0, st, p);
    else if (a_dtype == kF32 && w_dtype == kBF16) launch_kernel((grouped_rows_kernel<float, __nv_bfloat16, GATED>), grid, dim3(256), 0, st, p);
    else launch_kernel((grouped_rows_kernel<__nv_bfloat16, __nv_bfloat16, GATED>), grid, dim3(256), 0, st, p);
    return check_launch("grouped_product (rows)");
}

template <bool GATED>
static int launch_grouped(const GroupedArgs& p, int a_dtype, int w_dtype, dim3 grid, cudaStream_t st) {
    if (a_dtype == kF32 && w_dtype == kF32) launch_kernel((grouped_product_kernel<float, float, GATED>), grid, dim3(128), 0, st, p);
    else if (a_dtype == kF32 && w_dtype == kBF16) launch_kernel((grouped_product_kernel<float, __nv_bfloat16, GATED>), grid, dim3(128), 0, st, p);
    else if (a_dtype == kBF16 && w_dtype == kBF16) launch_kernel((grouped_product_kernel<__nv_bfloat16, __nv_bfloat16, GATED>), grid, dim3(128), 0, st, p);
    else { set_error("grouped_product: inputs of dtype code %d with weights of %d are not built", a_dtype, w_dtype); return 2; }
    return check_launch("grouped_product");
}

}  // namespace gi

using namespace gi;

extern "C" int gi_grouped_tile_rows() { return kGpTM; }

static int gi_head_product_impl(const void* a, int a_dtype, long long lda, int a_off, int a_gs, const void* w, int w_dtype,
                                long long w_gs, void* out, int out_dtype, long long ldo, int o_off, int o_gs, int rows, int heads,
                                int N, int K, int tail, const float* freq, float amplitude, const int* positions, const float* gate,
                                long long ldg, int gate_off, void* stream) {
    if (rows == 0) return 0;
    GI_REQUIRE(rows > 0 && heads > 0 && N > 0 && K > 0, "head_product: sizes must be positive");
    GI_REQUIRE(gate == nullptr || (gate_off >= 0 && gate_off + static_cast<long long>(heads) * N <= ldg), "head_product: the gate's columns lie outside its rows");
    GI_REQUIRE(tail >= 0 && tail % 2 == 0 && (tail == 0 || (freq && positions)), "head_product: a rotated tail needs an even size, frequencies and positions");
    GI_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "head_product: unsupported output dtype");
    GroupedArgs p = {};
    p.a = a; p.lda = lda; p.a_off = a_off; p.a_gs = a_gs; p.a_div = 1;
    p.w = w; p.w_gs = w_gs; p.ldw = K; p.up_off = 0;
    p.out = out; p.out_is_f32 = out_dtype == kF32; p.ldo = ldo; p.o_off = o_off; p.o_gs = o_gs;
    p.N = N; p.K = K; p.rows = rows; p.groups = heads;
    p.tail = tail; p.freq = freq; p.amplitude = amplitude; p.positions = positions;
    p.gate = gate; p.ldg = ldg; p.gate_off = gate_off;
    const long long tiles = static_cast<long long>((rows + kGpTM - 1) / kGpTM) * heads;
    GI_REQUIRE(tiles <= 2147483647LL, "head_product: too many tiles");
    dim3 grid(static_cast<unsigned>(tiles), (N + kGpTN - 1) / kGpTN);
    // many tokens: tiles of 64 x 64 where every group of four values is aligned (K in whole fours: no ragged piece)
    if (rows >= 2 * kG64 && K % 4 == 0 && lda % 4 == 0 && a_off % 4 == 0 && a_gs % 4 == 0 && w_gs % 4 == 0 &&
        reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 && !(a_dtype == kBF16 && w_dtype == kF32)) {
        const long long tiles64 = static_cast<long long>((rows + kG64 - 1) / kG64) * heads;
        GI_REQUIRE(tiles64 <= 2147483647LL, "head_product: too many tiles");
        dim3 grid64(static_cast<unsigned>(tiles64), (N + kG64 - 1) / kG64);
        cudaStream_t st64 = static_cast<cudaStream_t>(stream);
        if (a_dtype == kF32 && w_dtype == kF32) launch_kernel((head_product64_kernel<float, float>), grid64, dim3(256), 0, st64, p);
        else if (a_dtype == kF32) launch_kernel((head_product64_kernel<float, __nv_bfloat16>), grid64, dim3(256), 0, st64, p);
        else launch_kernel((head_product64_kernel<__nv_bfloat16, __nv_bfloat16>), grid64, dim3(256), 0, st64, p);
        return check_launch("head_product (tiles of 64)");
    }
    // few tokens: the heads' matrices are what is read; the rotated tail stays with the tiled form
    if (rows <= 2 * kGpTM && tail == 0 && rows_form_fits(p, a_dtype, w_dtype))
        return launch_grouped_rows<false>(p, a_dtype, w_dtype, static_cast<unsigned>(tiles), static_cast<cudaStream_t>(stream));
    return launch_grouped<false>(p, a_dtype, w_dtype, grid, static_cast<cudaStream_t>(stream));
}

static int gi_expert_product_impl(const void* a, int a_dtype, long long lda, int a_div, const void* w, int w_dtype, long long w_gs,
                                  int ldw, long long up_off, int gated, int act, float act_limit, void* out, int out_dtype, long long ldo,
                                  int N, int K, const int* tile_group, const int* sorted_rows, const int* n_tiles, int max_tiles,
                                  void* stream) {
    if (max_tiles == 0) return 0;
    GI_REQUIRE(max_tiles > 0 && N > 0 && K > 0 && a_div > 0, "expert_product: sizes must be positive");
    GI_REQUIRE(tile_group && sorted_rows && n_tiles, "expert_product: the sorted rows are missing");
    GI_REQUIRE(act >= 0 && act < kActCount, "expert_product: unknown activation code %d", act);
    GroupedArgs p = {};
    p.a = a; p.lda = lda; p.a_div = a_div;
    p.w = w; p.w_gs = w_gs; p.ldw = ldw; p.up_off = up_off;
    p.out = out; p.out_is_f32 = out_dtype == kF32; p.ldo = ldo;
    p.N = N; p.K = K; p.groups = 1;
    p.tile_group = tile_group; p.sorted_rows = sorted_rows; p.n_tiles = n_tiles; p.act = act; p.act_limit = act_limit;
    dim3 grid(max_tiles, (N + kGpTN - 1) / kGpTN);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows_form_fits(p, a_dtype, w_dtype))
        return gated ? launch_grouped_rows<true>(p, a_dtype, w_dtype, max_tiles, st) : launch_grouped_rows<false>(p, a_dtype, w_dtype, max_tiles, st);
    return gated ? launch_grouped<true>(p, a_dtype, w_dtype, grid, st) : launch_grouped<false>(p, a_dtype, w_dtype, grid, st);
}

static int gi_route_impl(const void* x, int x_dtype, int T, int D, const float* w, const float* correction, int E, int top,
                         int* ids, float* weights, int* sorted_rows, int* tile_group, int* n_tiles, int max_tiles, int tile_rows,
                         int* pair_row, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && D > 0 && E > 0 && top > 0 && top <= E, "route: sizes must be positive and top at most the experts");
    GI_REQUIRE(E <= kRouteMaxExperts, "route: %d experts exceed %d", E, kRouteMaxExperts);
    GI_REQUIRE(static_cast<size_t>(D) * 4 <= 160 * 1024, "route: a row of %d values does not fit shared memory", D);
    const long long pairs = static_cast<long long>(T) * top;
    GI_REQUIRE(tile_rows > 0, "route: tiles must have rows");
    GI_REQUIRE(max_tiles >= (pairs + tile_rows - 1) / tile_rows + std::min<long long>(E, pairs) - 1, "route: room for %d tiles is too little", max_tiles);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = static_cast<size_t>(D) * 4;
    if (x_dtype == kF32) {
        if (smem > 40 * 1024) cudaFuncSetAttribute(route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        launch_kernel((route_kernel<float>), dim3(T), dim3(128), smem, st, static_cast<const float*>(x), D, w, correction, E, top, ids, weights);
    } else if (x_dtype == kBF16) {
        if (smem > 40 * 1024) cudaFuncSetAttribute(route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        launch_kernel((route_kernel<__nv_bfloat16>), dim3(T), dim3(128), smem, st, static_cast<const __nv_bfloat16*>(x), D, w, correction, E, top, ids, weights);
    } else {
        GI_REQUIRE(false, "route: unsupported dtype code %d", x_dtype);
    }
    if (check_launch("route")) return 1;
    launch_kernel(route_align_kernel, dim3(1), dim3(1024), 0, st, static_cast<const int*>(ids), static_cast<int>(pairs), E, sorted_rows, tile_group, n_tiles, max_tiles, tile_rows, pair_row);
    return check_launch("route_align");
}

static int gi_route_table_impl(const int* tokens, const int* feedback, const int* table, int vocab, int T, int E, int top, int* ids,
                               float* weights, int* sorted_rows, int* tile_group, int* n_tiles, int max_tiles, int tile_rows,
                               int* pair_row, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && vocab > 0 && E > 0 && top > 0 && top <= E, "route_table: sizes must be positive and top at most the experts");
    GI_REQUIRE(E <= kRouteMaxExperts, "route_table: %d experts exceed %d", E, kRouteMaxExperts);
    const long long pairs = static_cast<long long>(T) * top;
    GI_REQUIRE(tile_rows > 0 && pairs <= 2147483647LL, "route_table: tiles must have rows");
    GI_REQUIRE(max_tiles >= (pairs + tile_rows - 1) / tile_rows + std::min<long long>(E, pairs) - 1, "route_table: room for %d tiles is too little", max_tiles);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    launch_kernel(route_table_kernel, dim3(static_cast<unsigned>((pairs + 255) / 256)), dim3(256), 0, st, tokens, feedback, table, vocab, E, top,
                  ids, weights, static_cast<int>(pairs));
    if (check_launch("route_table")) return 1;
    launch_kernel(route_align_kernel, dim3(1), dim3(1024), 0, st, static_cast<const int*>(ids), static_cast<int>(pairs), E, sorted_rows, tile_group, n_tiles, max_tiles, tile_rows, pair_row);
    return check_launch("route_align");
}

static int gi_gather_rows_impl(const void* x, int dtype, int D, int a_div, const int* sorted_rows, const int* n_tiles, int tile_rows,
                               int max_rows, void* out, void* stream) {
    if (max_rows == 0) return 0;
    GI_REQUIRE(max_rows > 0 && D > 0 && a_div > 0 && tile_rows > 0, "gather_rows: sizes must be positive");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == kBF16)
        launch_kernel((gather_rows_kernel<__nv_bfloat16>), dim3(max_rows), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), D, a_div,
                      sorted_rows, n_tiles, tile_rows, static_cast<__nv_bfloat16*>(out));
    else if (dtype == kF32)
        launch_kernel((gather_rows_kernel<float>), dim3(max_rows), dim3(256), 0, st, static_cast<const float*>(x), D, a_div, sorted_rows,
                      n_tiles, tile_rows, static_cast<float*>(out));
    else
        GI_REQUIRE(false, "gather_rows: unsupported dtype code %d", dtype);
    return check_launch("gather_rows");
}

static int gi_route_combine_impl(const float* part, const float* weights, const int* pair_row, float* y, int T, int D, int top, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && D > 0 && top > 0, "route_combine: sizes must be positive");
    const size_t total = static_cast<size_t>(T) * D;
    launch_kernel(route_combine_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  part, weights, pair_row, y, D, top, total);
    return check_launch("route_combine");
}

extern "C" int gi_head_product(const void* a, int a_dtype, long long lda, int a_off, int a_gs, const void* w, int w_dtype,
                               long long w_gs, void* out, int out_dtype, long long ldo, int o_off, int o_gs, int rows, int heads,
                               int N, int K, int tail, const float* freq, float amplitude, const int* positions, const float* gate,
                               long long ldg, int gate_off, void* stream) {
    return gi::dispatch(gi_head_product_impl, a, a_dtype, lda, a_off, a_gs, w, w_dtype, w_gs, out, out_dtype, ldo, o_off, o_gs, rows,
                        heads, N, K, tail, freq, amplitude, positions, gate, ldg, gate_off, stream);
}

extern "C" int gi_expert_product(const void* a, int a_dtype, long long lda, int a_div, const void* w, int w_dtype, long long w_gs,
                                 int ldw, long long up_off, int gated, int act, float act_limit, void* out, int out_dtype, long long ldo, int N, int K,
                                 const int* tile_group, const int* sorted_rows, const int* n_tiles, int max_tiles, void* stream) {
    return gi::dispatch(gi_expert_product_impl, a, a_dtype, lda, a_div, w, w_dtype, w_gs, ldw, up_off, gated, act, act_limit, out, out_dtype, ldo,
                        N, K, tile_group, sorted_rows, n_tiles, max_tiles, stream);
}

extern "C" int gi_route(const void* x, int x_dtype, int T, int D, const float* w, const float* correction, int E, int top, int* ids,
                        float* weights, int* sorted_rows, int* tile_group, int* n_tiles, int max_tiles, int tile_rows, int* pair_row,
                        void* stream) {
    return gi::dispatch(gi_route_impl, x, x_dtype, T, D, w, correction, E, top, ids, weights, sorted_rows, tile_group, n_tiles,
                        max_tiles, tile_rows, pair_row, stream);
}

extern "C" int gi_route_table(const int* tokens, const int* feedback, const int* table, int vocab, int T, int E, int top, int* ids,
                              float* weights, int* sorted_rows, int* tile_group, int* n_tiles, int max_tiles, int tile_rows,
                              int* pair_row, void* stream) {
    return gi::dispatch(gi_route_table_impl, tokens, feedback, table, vocab, T, E, top, ids, weights, sorted_rows, tile_group, n_tiles,
                        max_tiles, tile_rows, pair_row, stream);
}

extern "C" int gi_gather_rows(const void* x, int dtype, int D, int a_div, const int* sorted_rows, const int* n_tiles, int tile_rows,
                              int max_rows, void* out, void* stream) {
    return gi::dispatch(gi_gather_rows_impl, x, dtype, D, a_div, sorted_rows, n_tiles, tile_rows, max_rows, out, stream);
}

extern "C" int gi_route_combine(const float* part, const float* weights, const int* pair_row, float* y, int T, int D, int top, void* stream) {
    return gi::dispatch(gi_route_combine_impl, part, weights, pair_row, y, T, D, top, stream);
}
