// Mixers that carry a state of fixed size per request instead of keys and values: the recurrence
//
//     S_t = a_t S_(t-1) + b_t k_t v_t^T        (S: dk x dv per head, 32-bit, in the request's state slot)
//     o_t = S_t^T q_t + D v_t
//
// with its families of decay: a constant a per head and b = 1 (linear attention with decay);
// a_t = exp(-exp(A_log) dt_t), b_t = dt_t with dt_t = softplus(raw_t + bias) per head and token (state-space
// duality); and a factor of its own for every row of S, S_t = diag(alpha_t) S_(t-1) + k_t v_t^T with
// alpha_t = sigmoid(z_t)^(1/tau) per head, key channel and token (gated linear attention). Around it: the short causal convolution over a request's tokens whose last inputs are state too (with or without a bias
// and SiLU), and the unit-RMS norm over groups of channels with a gate before (SiLU) or after (sigmoid or SiLU) the norm.
//
// A step's rows are segments (one per request: seg_start, seg_len, state_slots as the step's descriptor holds
// them on the device). Tokens of a segment are taken in order, one after the other, by the same threads with the
// same arithmetic however the request was cut into steps and whatever else is in the batch; decays, step sizes,
// gates, norms and the state are 32-bit.
#include "common.cuh"

namespace gi {

__device__ __forceinline__ float silu_f(float z) { return z * (1.0f / (1.0f + expf(-z))); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------- causal convolution
// out[t, c] = act(bias[c] + sum_j w[c, j] * u(t - (taps-1) + j, c)), act SiLU or nothing, bias optional; u before the segment's first row is the
// request's conv state [taps-1, C] (oldest first; zeros for a new request), u before the sequence is zero.
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* __restrict__ in, int ld, int in_off, const float* __restrict__ weight,
                   const float* __restrict__ bias, const float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ row_req, const int* __restrict__ seg_start,
                   const int* __restrict__ state_slots, float* __restrict__ out, int C, int taps, int T, int act) {
    pdl_prologue();
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= C) return;
    const int r = row_req[t];
    const int rel = t - seg_start[r];
    const float* st = state + static_cast<long long>(state_slots[r]) * slot_stride;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                 // how many tokens before t
        float u;
        if (back <= rel) u = in[static_cast<size_t>(t - back) * ld + in_off + c];
        else u = st[static_cast<size_t>(taps - 1 + rel - back) * C + c];
        acc = fmaf(weight[static_cast<size_t>(c) * taps + j], u, acc);
    }
    out[static_cast<size_t>(t) * C + c] = act ? silu_f(acc) : acc;
}

// The state after the step: the last taps-1 inputs of each segment (older ones from the old state).
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const float* __restrict__ in, int ld, int in_off, float* __restrict__ state, long long slot_stride,
                         const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                         const int* __restrict__ state_slots, int C, int taps) {
    pdl_prologue();
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= C) return;
    const int n = seg_len[r], s0 = seg_start[r];
    float* st = state + static_cast<long long>(state_slots[r]) * slot_stride;
    const int keep = taps - 1;
    float vals[16];
    for (int j = 0; j < keep; ++j) {
        const int rel = n - keep + j;                 // index among the segment's rows; negative: old state
        vals[j] = rel >= 0 ? in[static_cast<size_t>(s0 + rel) * ld + in_off + c] : st[static_cast<size_t>(keep + rel) * C + c];
    }
    for (int j = 0; j < keep; ++j) st[static_cast<size_t>(j) * C + c] = vals[j];
}

// ---------------------------------------------------------------------------------- the recurrence
// A block owns 32 columns of one head's state of one request, each thread a few rows x 4 columns of it in registers.
// Tokens are staged a chunk at a time in shared memory (activated, with their a and b).
//
// Long segments are cut into parts of part_len tokens that run side by side (kParts): every part starts from a zero
// state and leaves its own end state U_p and, per token, the product A_t of the decays since the part's start
// (scan kernel); the parts' true start states follow from S_(p+1) = A_end(p) S_p + U_p, S_0 the request's state
// (link kernel, a short loop per state element); and every token gets what the start state adds to it,
// o_t += A_t S_p^T q_t (apply kernel, a small matrix product per part). Steps whose segments all fit one part run
// the scan kernel alone, straight on the state slot.
constexpr int kScanCols = 32;
constexpr int kScanChunk = 16;

struct ScanArgs {
    const float* q; const float* k; const float* v;      // rows of ld_q / ld_k / ld_v floats, at these column offsets
    int ld_q, ld_k, ld_v, q_off, k_off, v_off;
    int H, group;                                         // head h reads q/k head h / group
    int dk, dv;
    int act;                                              // 1: SiLU on q, k and v when they are read
    const float* decay;                                   // [H] constant decays, or null for the dt form
    const float* dt_raw; int ld_dt, dt_off;               // [T, ld_dt] at dt_off + h
    const float* dt_bias; const float* a_log; const float* skip;      // [H] each; skip may be null
    const float* gate_raw; int ld_gate, gate_off;         // [T, ld_gate] at gate_off + h * dk + i: z of the per-row decay, or null
    const float* gate_bias; float inv_tau;                // [H * dk] added to z (may be null); alpha = sigmoid(z)^inv_tau
    float q_scale;                                        // a constant on the queries
    float* state; long long slot_stride; long long state_off;          // per slot: [H, dk, dv] at state_off
    const int* seg_start; const int* seg_len; const int* state_slots;
    float* out;                                           // [T, H * dv]
    int part_len, max_parts;                              // kParts: tokens per part, parts per request in the grid
    float* ws_state;                                      // [parts of the step, H, dk, dv]
    float* ws_decay;                                      // [T, H]; with per-row decays [T, H, dk]
};

// sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
__device__ __forceinline__ float row_decay(float z, float inv_tau) { return expf(-softplus_f(-z) * inv_tau); }

// Where request r's parts start among the step's parts: the parts of the requests before it.
__device__ __forceinline__ int parts_before(const ScanArgs& p, int r) {
    int base = 0;
    for (int i = 0; i < r; ++i) base += (p.seg_len[i] + p.part_len - 1) / p.part_len;
    return base;
}

// (Left alone the compiler takes the kernel past 128 registers a thread, with a decay per row to 168, and a launch of a
// few heads' blocks then needs a second, nearly empty round over the SMs: it is held to 512 threads an SM.)
template <int kDk, int kRT, bool kParts, bool kRowDecay>
__global__ void __launch_bounds__(kDk / kRT * 8, (kRowDecay || kDk <= 128) ? 512 / (kDk / kRT * 8) : 1)
linear_scan_kernel(const ScanArgs p) {
    pdl_prologue();
    // A thread owns kRT rows x 4 columns of the state in registers (thread = row group x column group; a block covers
    // all kDk padded rows and 32 columns): per token it reads kRT k and q values and 4 v values from shared memory
    // for 4 kRT state elements. A token's output is the sum over the row groups, added up in their order once per
    // chunk of tokens.
    constexpr int kGroups = kDk / kRT;                    // row groups
    constexpr int kThreads = kGroups * 8;
    constexpr int kChunk = kDk >= 128 ? kScanChunk / 2 : kScanChunk;      // tokens staged at a time (shared memory)
    constexpr int kPerThread = kChunk * kDk / kThreads;   // q (and k) values a thread stages per chunk
    constexpr int kVPerThread = kChunk * kScanCols / kThreads;
    __shared__ __align__(16) float s_q[kChunk][kDk];
    __shared__ __align__(16) float s_k[kChunk][kDk];
    __shared__ __align__(16) float s_v[kChunk][kScanCols];
    __shared__ __align__(16) float s_o[kChunk][kGroups][kScanCols];
    __shared__ float s_a[kChunk], s_b[kChunk];
    __shared__ __align__(16) float s_av[kRowDecay ? kChunk : 1][kRowDecay ? kDk : 4];      // per-row decays of the staged tokens
    const int tile = blockIdx.x, h = blockIdx.y;
    const int r = kParts ? blockIdx.z / p.max_parts : blockIdx.z;
    const int part_idx = kParts ? blockIdx.z % p.max_parts : 0;
    const int g = h / p.group;
    const int cg = threadIdx.x % 8, rg = threadIdx.x / 8;
    const int j0 = tile * kScanCols + cg * 4;             // first of this thread's columns
    int n = p.seg_len[r], s0 = p.seg_start[r];
    float* S;
    if (kParts) {
        if (part_idx * p.part_len >= n) return;
        s0 += part_idx * p.part_len;
        n = min(p.part_len, n - part_idx * p.part_len);
        S = p.ws_state + (static_cast<size_t>(parts_before(p, r) + part_idx) * p.H + h) * p.dk * p.dv;
    } else {
        S = p.state + static_cast<long long>(p.state_slots[r]) * p.slot_stride + p.state_off +
            static_cast<long long>(h) * p.dk * p.dv;
    }
    float s[kRT][4];
#pragma unroll
    for (int i = 0; i < kRT; ++i) {
        const int row = rg * kRT + i;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            s[i][c] = (!kParts && row < p.dk && j0 + c < p.dv) ? S[static_cast<size_t>(row) * p.dv + j0 + c] : 0.f;
    }
    const float skip = p.skip ? p.skip[h] : 0.f;
    const float a_const = p.decay ? p.decay[h] : 0.f;
    const bool stepped = !kRowDecay && !p.decay;         // a and b from the step size
    const float neg_rate = stepped ? -expf(p.a_log[h]) : 0.f;
    const float bias = stepped ? p.dt_bias[h] : 0.f;
    float cum = 1.f;                                      // thread 0: product of the decays since the part's start
    constexpr int kCumPerThread = (kDk + kThreads - 1) / kThreads;
    float cumv[kCumPerThread];                            // per-row decays: the products of rows threadIdx.x + u * kThreads
#pragma unroll
    for (int u = 0; u < kCumPerThread; ++u) cumv[u] = 1.f;
    // the loads of a chunk are requested while the chunk before it is worked on
    float qv[kPerThread], kv[kPerThread], zv[kRowDecay ? kPerThread : 1], vv[kVPerThread], dt_raw = 0.f;
    auto request = [&](int c0) {
        const int m = min(kChunk, n - c0);
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            const int e = threadIdx.x + u * kThreads;
            const int tt = e / kDk, i = e % kDk;
            const size_t t = static_cast<size_t>(s0 + c0 + tt);
            const bool in = tt < m && i < p.dk;
            qv[u] = in ? p.q[t * p.ld_q + p.q_off + g * p.dk + i] : 0.f;
            kv[u] = in ? p.k[t * p.ld_k + p.k_off + g * p.dk + i] : 0.f;
            if (kRowDecay)
                zv[u] = in ? p.gate_raw[t * p.ld_gate + p.gate_off + h * p.dk + i] + (p.gate_bias ? p.gate_bias[h * p.dk + i] : 0.f) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < kVPerThread; ++u) {
            const int e = threadIdx.x + u * kThreads;
            const int tt = e / kScanCols, jj = tile * kScanCols + e % kScanCols;
            vv[u] = (tt < m && jj < p.dv) ? p.v[static_cast<size_t>(s0 + c0 + tt) * p.ld_v + p.v_off + h * p.dv + jj] : 0.f;
        }
        if (!kRowDecay && !p.decay && threadIdx.x < m)
            dt_raw = p.dt_raw[static_cast<size_t>(s0 + c0 + threadIdx.x) * p.ld_dt + p.dt_off + h];
    };
    request(0);
    for (int c0 = 0; c0 < n; c0 += kChunk) {
        const int m = min(kChunk, n - c0);
        __syncthreads();                                  // the chunk before is done with the staging buffers
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            const int e = threadIdx.x + u * kThreads;
            s_q[e / kDk][e % kDk] = (p.act ? silu_f(qv[u]) : qv[u]) * p.q_scale;
            s_k[e / kDk][e % kDk] = p.act ? silu_f(kv[u]) : kv[u];
            if (kRowDecay) s_av[e / kDk][e % kDk] = (e / kDk < m && e % kDk < p.dk) ? row_decay(zv[u], p.inv_tau) : 1.f;
        }
#pragma unroll
        for (int u = 0; u < kVPerThread; ++u) {
            const int e = threadIdx.x + u * kThreads;
            s_v[e / kScanCols][e % kScanCols] = p.act ? silu_f(vv[u]) : vv[u];
        }
        if (threadIdx.x < m) {
            if (kRowDecay) {
                s_a[threadIdx.x] = 1.f;
                s_b[threadIdx.x] = 1.f;
            } else if (p.decay) {
                s_a[threadIdx.x] = a_const;
                s_b[threadIdx.x] = 1.f;
            } else {
                const float dt = softplus_f(dt_raw + bias);
                s_a[threadIdx.x] = expf(neg_rate * dt);
                s_b[threadIdx.x] = dt;
            }
        }
        __syncthreads();
        if (c0 + kChunk < n) request(c0 + kChunk);
        if (kParts && !kRowDecay && tile == 0 && threadIdx.x == 0) {
            for (int tt = 0; tt < m; ++tt) {
                cum *= s_a[tt];
                p.ws_decay[static_cast<size_t>(s0 + c0 + tt) * p.H + h] = cum;
            }
        }
        if (kParts && kRowDecay && tile == 0) {
#pragma unroll
            for (int u = 0; u < kCumPerThread; ++u) {
                const int i = threadIdx.x + u * kThreads;
                if (i < p.dk) {
                    for (int tt = 0; tt < m; ++tt) {
                        cumv[u] *= s_av[tt][i];
                        p.ws_decay[(static_cast<size_t>(s0 + c0 + tt) * p.H + h) * p.dk + i] = cumv[u];
                    }
                }
            }
        }
        for (int tt = 0; tt < m; ++tt) {
            const float a = s_a[tt], b = s_b[tt];
            const float4 v4 = *reinterpret_cast<const float4*>(&s_v[tt][cg * 4]);
            const float bv[4] = {b * v4.x, b * v4.y, b * v4.z, b * v4.w};
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            const float4* k4 = reinterpret_cast<const float4*>(&s_k[tt][rg * kRT]);
            const float4* q4 = reinterpret_cast<const float4*>(&s_q[tt][rg * kRT]);
#pragma unroll
            for (int i4 = 0; i4 < kRT / 4; ++i4) {
                const float4 kk = k4[i4], qq = q4[i4];
                const float kr[4] = {kk.x, kk.y, kk.z, kk.w}, qr[4] = {qq.x, qq.y, qq.z, qq.w};
                float ar[4] = {a, a, a, a};
                if (kRowDecay) {
                    const float4 aa = reinterpret_cast<const float4*>(&s_av[tt][rg * kRT])[i4];
                    ar[0] = aa.x; ar[1] = aa.y; ar[2] = aa.z; ar[3] = aa.w;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        s[4 * i4 + u][c] = fmaf(ar[u], s[4 * i4 + u][c], kr[u] * bv[c]);
                        o[c] = fmaf(s[4 * i4 + u][c], qr[u], o[c]);
                    }
                }
            }
            *reinterpret_cast<float4*>(&s_o[tt][rg][cg * 4]) = make_float4(o[0], o[1], o[2], o[3]);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < m * kScanCols; e += kThreads) {
            const int tt = e / kScanCols, c = e % kScanCols;
            const int jj = tile * kScanCols + c;
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < kGroups; ++w) o += s_o[tt][w][c];
            if (jj < p.dv)
                p.out[static_cast<size_t>(s0 + c0 + tt) * p.H * p.dv + h * p.dv + jj] = fmaf(skip, s_v[tt][c], o);
        }
    }
#pragma unroll
    for (int i = 0; i < kRT; ++i) {
        const int row = rg * kRT + i;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (row < p.dk && j0 + c < p.dv) S[static_cast<size_t>(row) * p.dv + j0 + c] = s[i][c];
    }
}

// The parts' start states: one thread per element of a request's state walks over the request's parts.
__global__ void __launch_bounds__(256)
scan_link_kernel(const ScanArgs p) {
    pdl_prologue();
    const int r = blockIdx.y;
    const size_t per_head = static_cast<size_t>(p.dk) * p.dv;
    const size_t e = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
    if (e >= per_head * p.H) return;
    const int h = static_cast<int>(e / per_head);
    const int n = p.seg_len[r], s0 = p.seg_start[r];
    const int parts = (n + p.part_len - 1) / p.part_len;
    float* slot = p.state + static_cast<long long>(p.state_slots[r]) * p.slot_stride + p.state_off;
    float* ws = p.ws_state + static_cast<size_t>(parts_before(p, r)) * p.H * per_head;
    float S = slot[e];
    constexpr int kBatch = 8;                             // parts whose loads are in flight together
    for (int q0 = 0; q0 < parts; q0 += kBatch) {
        float U[kBatch], A[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int q = q0 + u;
            const bool in = q < parts;
            const int last = s0 + min((q + 1) * p.part_len, n) - 1;
            U[u] = in ? ws[static_cast<size_t>(q) * p.H * per_head + e] : 0.f;
            A[u] = !in ? 1.f : p.gate_raw ? p.ws_decay[(static_cast<size_t>(last) * p.H + h) * p.dk + (e % per_head) / p.dv]
                                          : p.ws_decay[static_cast<size_t>(last) * p.H + h];
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            if (q0 + u < parts) {
                ws[static_cast<size_t>(q0 + u) * p.H * per_head + e] = S;      // the state this part starts from
                S = fmaf(A[u], S, U[u]);
            }
        }
    }
    slot[e] = S;
}

// o_t += A_t S_p^T q_t for the tokens of one part, one head and 32 columns: the start state's columns and 16 tokens'
// queries (transposed) in shared memory, a warp per four tokens, a lane per column.
template <int kDk>
__global__ void __launch_bounds__(128)
scan_apply_kernel(const ScanArgs p) {
    pdl_prologue();
    constexpr int kChunk = kDk > 128 ? kScanChunk / 2 : kScanChunk;
    __shared__ float s_S[kDk][kScanCols];
    __shared__ __align__(16) float s_qT[kDk][kChunk + 4];      // rows 80 bytes apart: fewer bank conflicts when a chunk is laid down
    const int tile = blockIdx.x, h = blockIdx.y;
    const int r = blockIdx.z / p.max_parts, part_idx = blockIdx.z % p.max_parts;
    const int g = h / p.group;
    int n = p.seg_len[r], s0 = p.seg_start[r];
    if (part_idx * p.part_len >= n) return;
    s0 += part_idx * p.part_len;
    n = min(p.part_len, n - part_idx * p.part_len);
    const float* S = p.ws_state + (static_cast<size_t>(parts_before(p, r) + part_idx) * p.H + h) * p.dk * p.dv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = tile * kScanCols + lane;
    for (int e = threadIdx.x; e < kDk * kScanCols; e += 128) {
        const int i = e / kScanCols, jj = tile * kScanCols + e % kScanCols;
        s_S[i][e % kScanCols] = (i < p.dk && jj < p.dv) ? S[static_cast<size_t>(i) * p.dv + jj] : 0.f;
    }
    // the queries of a chunk are requested while the chunk before it is worked on
    constexpr int kPerThread = kChunk * kDk / 128;
    float qv[kPerThread], cv[kPerThread];
    auto request = [&](int c0) {
        const int m = min(kChunk, n - c0);
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            const int e = threadIdx.x + u * 128;
            const int tt = e / kDk, i = e % kDk;
            const bool in = tt < m && i < p.dk;
            qv[u] = in ? p.q[static_cast<size_t>(s0 + c0 + tt) * p.ld_q + p.q_off + g * p.dk + i] : 0.f;
            // per-row decays: the product since the part's start scales the query's own channel
            cv[u] = (in && p.gate_raw) ? p.ws_decay[(static_cast<size_t>(s0 + c0 + tt) * p.H + h) * p.dk + i] : 1.f;
        }
    };
    request(0);
    for (int c0 = 0; c0 < n; c0 += kChunk) {
        const int m = min(kChunk, n - c0);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            const int e = threadIdx.x + u * 128;
            s_qT[e % kDk][e / kDk] = (p.act ? silu_f(qv[u]) : qv[u]) * p.q_scale * cv[u];
        }
        __syncthreads();
        if (c0 + kChunk < n) request(c0 + kChunk);
        // what the sums are added to, and the decays that scale them, are on their way meanwhile
        float old[4], dec[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int tt = warp * 4 + u;
            const bool in = tt < m && j < p.dv;
            const size_t t = static_cast<size_t>(s0 + c0 + (in ? tt : 0));
            old[u] = in ? p.out[t * p.H * p.dv + h * p.dv + j] : 0.f;
            dec[u] = !in ? 0.f : p.gate_raw ? 1.f : p.ws_decay[t * p.H + h];
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (warp * 4 < kChunk)
#pragma unroll 8
        for (int i = 0; i < kDk; ++i) {
            const float sv = s_S[i][lane];
            const float4 q4 = *reinterpret_cast<const float4*>(&s_qT[i][warp * 4]);
            acc[0] = fmaf(q4.x, sv, acc[0]);
            acc[1] = fmaf(q4.y, sv, acc[1]);
            acc[2] = fmaf(q4.z, sv, acc[2]);
            acc[3] = fmaf(q4.w, sv, acc[3]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int tt = warp * 4 + u;
            if (tt < m && j < p.dv)
                p.out[static_cast<size_t>(s0 + c0 + tt) * p.H * p.dv + h * p.dv + j] = fmaf(dec[u], acc[u], old[u]);
        }
    }
}

// ---------------------------------------------------------------------------------- gated group norm
// One block per (token, group). mode 0: out = w * unit_rms(y) * sigmoid(gate); mode 1: out = w * unit_rms(y * silu(gate));
// mode 2: out = w * unit_rms(y) * silu(gate).
// Groups of at most 4096 channels in 16-byte pieces (kVec) are read once and kept in registers between the sum
// and the scaling; the sum's order (a fixed strided assignment, a fixed xor tree, the warps in index order) is
// the same in both forms.
template <typename TOut, bool kVec>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ld_gate, int gate_off,
                        const float* __restrict__ weight, TOut* __restrict__ out, int W, int groups, float eps,
                        int mode, float out_scale) {
    pdl_prologue();
    __shared__ float warp_part[8];
    const int t = blockIdx.x, grp = blockIdx.y;
    const int n = W / groups;
    const float* yr = y + static_cast<size_t>(t) * W + grp * n;
    const float* gr = gate + static_cast<size_t>(t) * ld_gate + gate_off + grp * n;
    TOut* o = out + static_cast<size_t>(t) * W + grp * n;
    const float* w = weight + grp * n;
    float ss = 0.f;
    float4 kept[4], gk[4];
    if (kVec) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x + k * 256;
            kept[k] = gk[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < n / 4) {
                kept[k] = reinterpret_cast<const float4*>(yr)[i];
                gk[k] = reinterpret_cast<const float4*>(gr)[i];
                if (mode == 1) {
                    kept[k].x *= silu_f(gk[k].x); kept[k].y *= silu_f(gk[k].y);
                    kept[k].z *= silu_f(gk[k].z); kept[k].w *= silu_f(gk[k].w);
                }
            }
            ss = fmaf(kept[k].x, kept[k].x, ss); ss = fmaf(kept[k].y, kept[k].y, ss);
            ss = fmaf(kept[k].z, kept[k].z, ss); ss = fmaf(kept[k].w, kept[k].w, ss);
        }
    } else {
        for (int d = threadIdx.x; d < n; d += 256) {
            const float v = mode == 1 ? yr[d] * silu_f(gr[d]) : yr[d];
            ss = fmaf(v, v, ss);
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += warp_part[k];
    const float scale = 1.0f / sqrtf(total / static_cast<float>(n) + eps);
    if (kVec) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i >= n / 4) continue;
            const float4 ww = reinterpret_cast<const float4*>(w)[i];
            float r[4] = {ww.x * (scale * kept[k].x), ww.y * (scale * kept[k].y), ww.z * (scale * kept[k].z), ww.w * (scale * kept[k].w)};
            if (mode == 0) {
                r[0] *= 1.0f / (1.0f + expf(-gk[k].x)); r[1] *= 1.0f / (1.0f + expf(-gk[k].y));
                r[2] *= 1.0f / (1.0f + expf(-gk[k].z)); r[3] *= 1.0f / (1.0f + expf(-gk[k].w));
            } else if (mode == 2) {
                r[0] *= silu_f(gk[k].x); r[1] *= silu_f(gk[k].y); r[2] *= silu_f(gk[k].z); r[3] *= silu_f(gk[k].w);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) o[4 * i + c] = from_float<TOut>(r[c] * out_scale);
        }
    } else {
        for (int d = threadIdx.x; d < n; d += 256) {
            float v;
            if (mode == 1) v = w[d] * (scale * (yr[d] * silu_f(gr[d])));
            else if (mode == 2) v = w[d] * (scale * yr[d]) * silu_f(gr[d]);
            else v = w[d] * (scale * yr[d]) * (1.0f / (1.0f + expf(-gr[d])));
            o[d] = from_float<TOut>(v * out_scale);
        }
    }
}

// The same for groups of at most 512 channels in 16-byte pieces: a warp per (token, group), eight groups a block, no
// block barrier; a lane keeps its up to four pieces in registers. The sum's order: a lane's chain over its pieces, then
// the fixed xor tree.
template <typename TOut>
__global__ void __launch_bounds__(256)
gated_group_norm_warp_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ld_gate, int gate_off,
                             const float* __restrict__ weight, TOut* __restrict__ out, int W, int groups, float eps,
                             int mode, float out_scale, long long total_groups) {
    pdl_prologue();
    const long long item = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (item >= total_groups) return;
    const int lane = threadIdx.x & 31;
    const long long t = item / groups;
    const int grp = static_cast<int>(item % groups);
    const int n = W / groups;
    const float4* yr = reinterpret_cast<const float4*>(y + static_cast<size_t>(t) * W + grp * n);
    const float4* gr = reinterpret_cast<const float4*>(gate + static_cast<size_t>(t) * ld_gate + gate_off + grp * n);
    const float4* w = reinterpret_cast<const float4*>(weight + grp * n);
    TOut* o = out + static_cast<size_t>(t) * W + grp * n;
    float4 kept[4], gk[4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = lane + k * 32;
        kept[k] = gk[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n / 4) {
            kept[k] = yr[i];
            gk[k] = gr[i];
            if (mode == 1) {
                kept[k].x *= silu_f(gk[k].x); kept[k].y *= silu_f(gk[k].y);
                kept[k].z *= silu_f(gk[k].z); kept[k].w *= silu_f(gk[k].w);
            }
        }
        ss = fmaf(kept[k].x, kept[k].x, ss); ss = fmaf(kept[k].y, kept[k].y, ss);
        ss = fmaf(kept[k].z, kept[k].z, ss); ss = fmaf(kept[k].w, kept[k].w, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = lane + k * 32;
        if (i >= n / 4) continue;
        const float4 ww = w[i];
        float r[4] = {ww.x * (scale * kept[k].x), ww.y * (scale * kept[k].y), ww.z * (scale * kept[k].z), ww.w * (scale * kept[k].w)};
        if (mode == 0) {
            r[0] *= 1.0f / (1.0f + expf(-gk[k].x)); r[1] *= 1.0f / (1.0f + expf(-gk[k].y));
            r[2] *= 1.0f / (1.0f + expf(-gk[k].z)); r[3] *= 1.0f / (1.0f + expf(-gk[k].w));
        } else if (mode == 2) {
            r[0] *= silu_f(gk[k].x); r[1] *= silu_f(gk[k].y); r[2] *= silu_f(gk[k].z); r[3] *= silu_f(gk[k].w);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) o[4 * i + c] = from_float<TOut>(r[c] * out_scale);
    }
}

}  // namespace gi

using namespace gi;

static int gi_causal_conv_impl(const float* in, int ld, int in_off, const float* weight, const float* bias, float* state,
                               long long slot_stride, long long state_off, const int* row_req, const int* seg_start,
                               const int* seg_len, const int* state_slots, float* out, int C, int taps, int T, int R,
                               int act, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && R > 0 && C > 0, "causal_conv: sizes must be positive");
    GI_REQUIRE(taps >= 1 && taps <= 17, "causal_conv: %d taps are not supported (1 to 17)", taps);
    GI_REQUIRE(T <= 65535 && R <= 65535, "causal_conv: %d rows in one step exceed the grid limit 65535", T);
    GI_REQUIRE(in_off >= 0 && in_off + C <= ld, "causal_conv: the channels lie outside the input row of %d", ld);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned cb = (C + 255) / 256;
    launch_kernel((causal_conv_kernel), dim3(cb, T), dim3(256), 0, st, in, ld, in_off, weight, bias,
                  static_cast<const float*>(state + state_off), slot_stride, row_req, seg_start, state_slots, out, C, taps, T, act);
    if (taps > 1)
        launch_kernel((conv_state_update_kernel), dim3(cb, R), dim3(256), 0, st, in, ld, in_off, state + state_off, slot_stride,
                      seg_start, seg_len, state_slots, C, taps);
    return check_launch("causal_conv");
}

template <int kDk, int kRT>
static void launch_scan(const ScanArgs& a, int R, cudaStream_t st) {
    const unsigned tiles = (a.dv + kScanCols - 1) / kScanCols;
    constexpr int kThreads = kDk / kRT * 8;
    const bool rows = a.gate_raw != nullptr;
    if (a.part_len == 0) {
        if (rows) launch_kernel((linear_scan_kernel<kDk, kRT, false, true>), dim3(tiles, a.H, R), dim3(kThreads), 0, st, a);
        else launch_kernel((linear_scan_kernel<kDk, kRT, false, false>), dim3(tiles, a.H, R), dim3(kThreads), 0, st, a);
        return;
    }
    if (rows) launch_kernel((linear_scan_kernel<kDk, kRT, true, true>), dim3(tiles, a.H, R * a.max_parts), dim3(kThreads), 0, st, a);
    else launch_kernel((linear_scan_kernel<kDk, kRT, true, false>), dim3(tiles, a.H, R * a.max_parts), dim3(kThreads), 0, st, a);
    const size_t elements = static_cast<size_t>(a.H) * a.dk * a.dv;
    launch_kernel((scan_link_kernel), dim3(static_cast<unsigned>((elements + 255) / 256), R), dim3(256), 0, st, a);
    launch_kernel((scan_apply_kernel<kDk>), dim3(tiles, a.H, R * a.max_parts), dim3(128), 0, st, a);
}

// part_len 0: every segment is walked from the request's state by one block per head and column tile. Otherwise
// segments are cut into parts of part_len tokens (at most max_parts per request) that run side by side; ws_state
// holds [parts of the step, H, dk, dv] floats and ws_decay [T, H].
static int gi_linear_scan_impl(const float* q, int ld_q, int q_off, const float* k, int ld_k, int k_off, const float* v,
                               int ld_v, int v_off, int H, int group, int dk, int dv, int act, const float* decay,
                               const float* dt_raw, int ld_dt, int dt_off, const float* dt_bias, const float* a_log,
                               const float* skip, const float* gate_raw, int ld_gate, int gate_off, const float* gate_bias,
                               float inv_tau, float q_scale, float* state, long long slot_stride, long long state_off,
                               const int* seg_start, const int* seg_len, const int* state_slots, float* out, int R,
                               int part_len, int max_parts, float* ws_state, float* ws_decay, void* stream) {
    if (R == 0) return 0;
    GI_REQUIRE(R > 0 && H > 0 && dk > 0 && dv > 0 && group > 0, "linear_scan: sizes must be positive");
    GI_REQUIRE(H % group == 0, "linear_scan: %d heads are not a multiple of the group size %d", H, group);
    GI_REQUIRE(dk <= 256, "linear_scan: %d state rows per head exceed 256", dk);
    GI_REQUIRE(decay != nullptr || gate_raw != nullptr || (dt_raw != nullptr && dt_bias != nullptr && a_log != nullptr),
               "linear_scan: neither constant decays nor step sizes nor per-row decays are given");
    GI_REQUIRE(gate_raw == nullptr || (group == 1 && gate_off >= 0 && gate_off + H * dk <= ld_gate),
               "linear_scan: per-row decays need a key head per head and their columns inside a row of %d", ld_gate);
    GI_REQUIRE(part_len == 0 || (part_len > 0 && max_parts > 0 && ws_state != nullptr && ws_decay != nullptr),
               "linear_scan: parts need their length, their number and both workspaces");
    GI_REQUIRE(static_cast<long long>(R) * (part_len ? max_parts : 1) <= 65535 && H <= 65535, "linear_scan: the grid limit 65535 is exceeded");
    ScanArgs a{q, k, v, ld_q, ld_k, ld_v, q_off, k_off, v_off, H, group, dk, dv, act, decay, dt_raw, ld_dt, dt_off, dt_bias,
               a_log, skip, gate_raw, ld_gate, gate_off, gate_bias, inv_tau, q_scale, state, slot_stride, state_off, seg_start, seg_len, state_slots, out, part_len, max_parts, ws_state,
               ws_decay};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // (padded state rows, rows per thread)
    if (dk <= 16) launch_scan<16, 4>(a, R, st);
    else if (dk <= 32) launch_scan<32, 4>(a, R, st);
    else if (dk <= 64) launch_scan<64, 8>(a, R, st);
    else if (dk <= 128) launch_scan<128, 8>(a, R, st);
    else launch_scan<256, 16>(a, R, st);
    return check_launch("linear_scan");
}

static int gi_gated_group_norm_impl(const float* y, const float* gate, int ld_gate, int gate_off, const float* weight, void* out,
                                    int out_dtype, int T, int W, int groups, float eps, int mode, float out_scale, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && W > 0 && groups > 0 && W % groups == 0, "gated_group_norm: %d channels do not split into %d groups", W, groups);
    GI_REQUIRE(T <= 2147483647 && groups <= 65535, "gated_group_norm: the grid limit is exceeded");
    GI_REQUIRE(mode >= 0 && mode <= 2, "gated_group_norm: unknown mode %d", mode);
    GI_REQUIRE(gate_off >= 0 && gate_off + W <= ld_gate, "gated_group_norm: the gate lies outside its row of %d", ld_gate);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int n = W / groups;
    const bool vec = n % 4 == 0 && n <= 4096 && W % 4 == 0 && ld_gate % 4 == 0 && gate_off % 4 == 0 &&
                     reinterpret_cast<uintptr_t>(y) % 16 == 0 && reinterpret_cast<uintptr_t>(gate) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(weight) % 16 == 0;
    if (vec && n <= 512 && groups > 1 && (out_dtype == kBF16 || out_dtype == kF32)) {
        // small groups: a warp per group
        const long long total = static_cast<long long>(T) * groups;
        const unsigned blocks = static_cast<unsigned>((total + 7) / 8);
        if (out_dtype == kBF16) launch_kernel((gated_group_norm_warp_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight, static_cast<__nv_bfloat16*>(out), W, groups, eps, mode, out_scale, total);
        else launch_kernel((gated_group_norm_warp_kernel<float>), dim3(blocks), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight, static_cast<float*>(out), W, groups, eps, mode, out_scale, total);
        return check_launch("gated_group_norm");
    }
    if (out_dtype == kBF16) {
        if (vec) launch_kernel((gated_group_norm_kernel<__nv_bfloat16, true>), dim3(T, groups), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight, static_cast<__nv_bfloat16*>(out), W, groups, eps, mode, out_scale);
        else launch_kernel((gated_group_norm_kernel<__nv_bfloat16, false>), dim3(T, groups), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight, static_cast<__nv_bfloat16*>(out), W, groups, eps, mode, out_scale);
    } else if (out_dtype == kF32) {
        if (vec) launch_kernel((gated_group_norm_kernel<float, true>), dim3(T, groups), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight, static_cast<float*>(out), W, groups, eps, mode, out_scale);
        else launch_kernel((gated_group_norm_kernel<float, false>), dim3(T, groups), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight, static_cast<float*>(out), W, groups, eps, mode, out_scale);
    }
    else
        GI_REQUIRE(false, "gated_group_norm: unsupported output dtype code %d", out_dtype);
    return check_launch("gated_group_norm");
}

extern "C" int gi_causal_conv(const float* in, int ld, int in_off, const float* weight, const float* bias, float* state, long long slot_stride, long long state_off, const int* row_req, const int* seg_start, const int* seg_len, const int* state_slots, float* out, int C, int taps, int T, int R, int act, void* stream) {
    return gi::dispatch(gi_causal_conv_impl, in, ld, in_off, weight, bias, state, slot_stride, state_off, row_req, seg_start, seg_len, state_slots, out, C, taps, T, R, act, stream);
}

extern "C" int gi_linear_scan(const float* q, int ld_q, int q_off, const float* k, int ld_k, int k_off, const float* v, int ld_v, int v_off, int H, int group, int dk, int dv, int act, const float* decay, const float* dt_raw, int ld_dt, int dt_off, const float* dt_bias, const float* a_log, const float* skip, const float* gate_raw, int ld_gate, int gate_off, const float* gate_bias, float inv_tau, float q_scale, float* state, long long slot_stride, long long state_off, const int* seg_start, const int* seg_len, const int* state_slots, float* out, int R, int part_len, int max_parts, float* ws_state, float* ws_decay, void* stream) {
    return gi::dispatch(gi_linear_scan_impl, q, ld_q, q_off, k, ld_k, k_off, v, ld_v, v_off, H, group, dk, dv, act, decay, dt_raw, ld_dt, dt_off, dt_bias, a_log, skip, gate_raw, ld_gate, gate_off, gate_bias, inv_tau, q_scale, state, slot_stride, state_off, seg_start, seg_len, state_slots, out, R, part_len, max_parts, ws_state, ws_decay, stream);
}

extern "C" int gi_gated_group_norm(const float* y, const float* gate, int ld_gate, int gate_off, const float* weight, void* out, int out_dtype, int T, int W, int groups, float eps, int mode, float out_scale, void* stream) {
    return gi::dispatch(gi_gated_group_norm_impl, y, gate, ld_gate, gate_off, weight, out, out_dtype, T, W, groups, eps, mode, out_scale, stream);
}
