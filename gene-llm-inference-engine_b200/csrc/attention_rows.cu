// Paged attention, row form with shared key tiles: one block per (query row, key/value head, group of query heads).
// The block brings tiles of 32 keys (and their values) into shared memory once and every warp of the block works on
// query heads of its own over them, so the heads of a group read their keys once and no results of different warps
// have to be merged. All arithmetic is 32-bit, also where the cache is bfloat16; queries are 32-bit or bfloat16.
//
// What a row sees and how a score is made are parameters:
//   window   w > 0: the query at position P sees keys P-w+1 .. P
//   chunk    c > 0: only keys of the query's own block of c positions counted from 0, floor(j / c) = floor(P / c)
//   slopes   [H] or null: slope_h * (P - j) is taken off the score of key j (a bias that grows with the distance)
//   sinks    [H] or null: the softmax's denominator also holds exp(sinks_h), a term without key or value
//   softcap  c > 0: the scaled score s becomes c tanh(s / c) before bias and softmax
//   values   a width ``vd`` of their own; they may lie in pages of their own or be the first vd columns of the key
//            rows (``v_row`` is the length of the rows they lie in), which serves attention over a shared latent whose
//            keys are [latent, rotated part] and whose values are the latent itself
// The online softmax walks the keys in tiles counted from the row's first visible key, so a row's result depends on
// that row's query, position and cache contents only.
#include "common.cuh"

namespace gi {

constexpr int kRowsTile = 32;        // keys per tile: one per lane

template <typename T> struct Pair2;
template <> struct Pair2<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Pair2<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
};

struct RowsArgs {
    const void* q; int q_is_f32; int ldq;          // queries [T, ldq], head h at column h * hd
    const void* k_cache; const void* v_cache;      // [pages, Hkv, page_size, hd] and [pages, Hkv, page_size, v_row]
    void* out; int out_is_f32; int ldo;            // [T, ldo], head h at column h * vd
    const int* row_req; const int* positions; const int* block_tables; int table_stride;
    int H, Hkv, hd, vd, v_row, page_size;
    float scale; float softcap; int window, chunk;
    const float* slopes; const float* sinks;
    int heads_per_block;                           // query heads of one key/value head that a block takes
    int ks;                                        // row length of the key tile in shared memory (elements)
    int alias;                                     // the values are the first vd columns of the key rows
};

__device__ __forceinline__ float capped(float score, float cap) { return cap > 0.f ? cap * tanhf(score / cap) : score; }

// HPW: query heads per warp; VI: value dimensions per lane (vd <= 32 * VI).
template <typename T, int HPW, int VI>
__global__ void __launch_bounds__(128)
attention_rows_kernel(const RowsArgs a) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int t = blockIdx.x, g = blockIdx.y;
    const int group = a.H / a.Hkv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hdp = (a.hd + 1) & ~1;
    const int first_head = blockIdx.z * a.heads_per_block;        // within the group
    const int n_heads = min(a.heads_per_block, group - first_head);

    float* s_q = reinterpret_cast<float*>(smem_raw);                              // [heads_per_block][hdp]
    T* s_k = reinterpret_cast<T*>(s_q + a.heads_per_block * hdp);                  // [32][ks]
    T* s_v = a.alias ? s_k : s_k + kRowsTile * a.ks;                               // [32][vd]
    const int vs = a.alias ? a.ks : a.vd;

    const int pos = a.positions[t];
    int lo = 0;
    if (a.window > 0) lo = max(lo, pos - a.window + 1);
    if (a.chunk > 0) lo = max(lo, pos / a.chunk * a.chunk);
    const int* table = a.block_tables + static_cast<size_t>(a.row_req[t]) * a.table_stride;

    // the block's queries, 32-bit; an odd head size is padded with a zero
    for (int i = threadIdx.x; i < n_heads * hdp; i += blockDim.x) {
        const int hh = i / hdp, d = i % hdp;
        float v = 0.f;
        if (d < a.hd) {
            const size_t off = static_cast<size_t>(t) * a.ldq + static_cast<size_t>(g * group + first_head + hh) * a.hd + d;
            v = a.q_is_f32 ? static_cast<const float*>(a.q)[off] : to_float(static_cast<const __nv_bfloat16*>(a.q)[off]);
        }
        s_q[i] = v;
    }

    float acc[HPW][VI];
    float m[HPW], l[HPW], slope[HPW];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        m[hh] = -INFINITY; l[hh] = 0.f;
        const int head = first_head + warp * HPW + hh;
        slope[hh] = (a.slopes && head < group) ? a.slopes[g * group + head] : 0.f;
#pragma unroll
        for (int i = 0; i < VI; ++i) acc[hh][i] = 0.f;
    }
    const bool warp_active = warp * HPW < n_heads;
    const T* kc = static_cast<const T*>(a.k_cache);
    const T* vc = static_cast<const T*>(a.v_cache);

    for (int base = lo; base <= pos; base += kRowsTile) {
        const int n_keys = min(kRowsTile, pos - base + 1);
        __syncthreads();                       // the tile before is done with (and the queries are written)
        // every warp fetches keys of its own: key j of the tile lands in row j (lane j looks up key j's page row, so the
        // look-ups of a tile are in flight together)
        size_t my_row = 0;
        if (lane < n_keys) {
            const int pl = base + lane;
            my_row = (static_cast<size_t>(table[pl / a.page_size]) * a.Hkv + g) * a.page_size + (pl % a.page_size);
        }
        for (int j = warp; j < n_keys; j += blockDim.x >> 5) {
            const size_t row = __shfl_sync(0xffffffffu, static_cast<unsigned long long>(my_row), j);
            const T* src = kc + row * a.hd;
            T* dst = s_k + j * a.ks;
            for (int d = lane; d < hdp; d += 32) dst[d] = d < a.hd ? src[d] : from_float<T>(0.f);
            if (!a.alias) {
                const T* vsrc = vc + row * a.v_row;
                T* vdst = s_v + j * a.vd;
                for (int d = lane; d < a.vd; d += 32) vdst[d] = vsrc[d];
            }
        }
        __syncthreads();
        if (!warp_active) continue;
        // scores: a lane per key, the block's heads one after the other over the same key row
        float s[HPW];
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) s[hh] = 0.f;
        const bool valid = lane < n_keys;
        if (valid) {
            const T* krow = s_k + lane * a.ks;
            for (int d = 0; d < hdp; d += 2) {
                const float2 kk = Pair2<T>::load(krow + d);
#pragma unroll
                for (int hh = 0; hh < HPW; ++hh) {
                    const float2 qq = *reinterpret_cast<const float2*>(s_q + (warp * HPW + hh) * hdp + d);
                    s[hh] = fmaf(qq.x, kk.x, s[hh]);
                    s[hh] = fmaf(qq.y, kk.y, s[hh]);
                }
            }
        }
        float p[HPW];
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const float score = valid ? capped(s[hh] * a.scale, a.softcap) - slope[hh] * static_cast<float>(pos - (base + lane)) : -INFINITY;
            const float m_new = fmaxf(m[hh], warp_max(score));          // finite: a tile always holds a visible key
            p[hh] = valid ? expf(score - m_new) : 0.f;
            const float corr = (m[hh] == -INFINITY) ? 0.f : expf(m[hh] - m_new);
            l[hh] = l[hh] * corr + warp_sum(p[hh]);
#pragma unroll
            for (int i = 0; i < VI; ++i) acc[hh][i] *= corr;
            m[hh] = m_new;
        }
        for (int j = 0; j < n_keys; ++j) {
            float pj[HPW];
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) pj[hh] = __shfl_sync(0xffffffffu, p[hh], j);
            const T* vrow = s_v + j * vs;
#pragma unroll
            for (int i = 0; i < VI; ++i) {
                const int d = lane + 32 * i;
                if (d < a.vd) {
                    const float v = to_float(vrow[d]);
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) acc[hh][i] = fmaf(pj[hh], v, acc[hh][i]);
                }
            }
        }
    }

    if (!warp_active) return;
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int head = first_head + warp * HPW + hh;
        if (head >= group) continue;
        const int h = g * group + head;
        float M = m[hh], L = l[hh], f = 1.f;
        if (a.sinks) {
            const float sk = a.sinks[h];
            M = fmaxf(M, sk);
            f = expf(m[hh] - M);
            L = L * f + expf(sk - M);
        }
        const float mul = f / L;
        const size_t o = static_cast<size_t>(t) * a.ldo + static_cast<size_t>(h) * a.vd;
#pragma unroll
        for (int i = 0; i < VI; ++i) {
            const int d = lane + 32 * i;
            if (d < a.vd) {
                const float v = acc[hh][i] * mul;
                if (a.out_is_f32) static_cast<float*>(a.out)[o + d] = v;
                else static_cast<__nv_bfloat16*>(a.out)[o + d] = __float2bfloat16_rn(v);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ tensor cores
// The same attention for a bfloat16 cache on the tensor cores (mma.sync m16n8k16): one block per (tile of query rows,
// key/value head, block of query heads, range of the keys). The sixteen rows of an MMA tile are the query heads of a
// group: all sixteen of one token where a key/value head serves sixteen or more heads (attention over a shared latent:
// all heads read one row per key), or the heads of several consecutive tokens of one request where it serves fewer
// (16 / group tokens; every row has its own position and so its own first and last visible key). Key tiles of 32 rows
// come through cp.async into two stages; the four warps share a tile's work: each takes every fourth 16-wide slice of
// the head dimension of S = Q K^T (the partial sums meet in shared memory and are added in warp order) and a quarter of
// the value dimensions of O += P V, so the accumulators of a 512-wide value are 64 registers a thread. Scores,
// softmax, bias and sinks are 32-bit as above; queries and the softmax's weights are rounded to bfloat16 where they
// enter a product. With few tiles (decoding) the keys are cut into ``splits`` ranges that run side by side and leave
// unnormalised sums, maxima and weights in a workspace, which a second kernel merges in the ranges' order.
__device__ __forceinline__ void rows_cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void rows_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void rows_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void rows_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void rows_ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void rows_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t rows_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t rows_smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

constexpr int kMmaHeads = 16;          // rows of an MMA tile
constexpr int kMmaOwnRows = 64;        // rows of a block whose warps each own an MMA tile of rows (small heads)
constexpr int kMmaPad = 8;             // bfloat16 values of padding per row of a tile (16 bytes: ldmatrix without conflicts)
constexpr int kMmaSStride = kRowsTile + 8;     // 40 floats: pairs of columns read by half a warp fall into different banks

// Which rows of the step a block works on: tile b of the list.
struct RowTiles {
    const int* list;       // kind 1: the row of tile b; kind 2: (first row, tokens, request) of tile b; kind 0: tile b = row b
    int kind;
    int head_blocks;       // blocks of sixteen heads per key/value head (groups of more than sixteen heads)
    int splits;            // ranges of keys that run side by side (> 1: results go through ``workspace``)
    int block_rows;        // query rows of a block: 16 (the warps share them) or 64 (a warp owns 16)
    float* workspace;      // [tiles][Hkv][head_blocks][splits][block_rows][vd + 2]
};

struct TileRows {
    int row0, ntok, gp;
    __device__ __forceinline__ int token(int r) const { return r / gp; }
    __device__ __forceinline__ int head(int r) const { return r % gp; }
};
__device__ __forceinline__ TileRows tile_rows(const RowTiles& rt, int b, int group) {
    TileRows t;
    if (rt.kind == 2) { t.row0 = rt.list[3 * b]; t.ntok = rt.list[3 * b + 1]; }
    else { t.row0 = rt.kind == 1 ? rt.list[b] : b; t.ntok = 1; }
    t.gp = min(group, kMmaHeads);
    return t;
}
__device__ __forceinline__ int first_visible(const RowsArgs& a, int pos) {
    int lo = 0;
    if (a.window > 0) lo = max(lo, pos - a.window + 1);
    if (a.chunk > 0) lo = max(lo, pos / a.chunk * a.chunk);
    return lo;
}

// NV: 8-wide tiles of value dimensions per warp. MODE 0: the four warps share sixteen rows, each with a quarter of the
// head dimension of S and of the value dimensions (vd <= 32 NV). MODE 1 (head and value sizes up to 128, groups of at
// most sixteen heads): every warp owns sixteen of the block's 64 rows, with all of the head dimension and all value
// dimensions (vd <= 8 NV), so the warps exchange nothing. MODE 2 (sixteen or more heads to a key/value head, large
// heads: the latent): two tokens of sixteen heads a block, two warps a token; each computes all of S for its token (the
// price: S twice) and keeps half of the value dimensions (vd <= 16 NV), so again nothing is exchanged and two tokens
// share every key tile.
template <int NV, int MODE>
__global__ void __launch_bounds__(128)
attention_rows_mma_kernel(const RowsArgs a, const RowTiles rt) {
    constexpr bool OWN = MODE == 1, PAIR = MODE == 2;
    constexpr int RT = OWN ? kMmaOwnRows : PAIR ? 2 * kMmaHeads : kMmaHeads;
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    using bf = __nv_bfloat16;
    const int g = blockIdx.y;
    const int group = a.H / a.Hkv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int zb = blockIdx.z % rt.head_blocks, split = blockIdx.z / rt.head_blocks;
    const TileRows tr = tile_rows(rt, blockIdx.x, group);
    const int first_head = zb * kMmaHeads;
    const int n_heads = min(kMmaHeads, group - first_head);
    const int n_rows = (!OWN && tr.gp == kMmaHeads) ? n_heads : tr.ntok * tr.gp;
    auto row_on = [&](int r) { return PAIR ? ((r >> 4) < tr.ntok && (r & 15) < n_heads) : r < n_rows; };
    const int qs = a.hd + kMmaPad;                     // row length of the query and key tiles
    const int vs = a.alias ? qs : a.vd + kMmaPad;
    bf* s_q = reinterpret_cast<bf*>(smem_raw);                              // [16][qs]
    bf* s_k = s_q + RT * qs;                                                // [2][32][qs]
    bf* s_v = a.alias ? s_k : s_k + 2 * kRowsTile * qs;                     // [2][32][vs]
    float* s_s = reinterpret_cast<float*>(s_k + 2 * kRowsTile * qs + (a.alias ? 0 : 2 * kRowsTile * vs));   // [4][16][36]

    const int pos0 = a.positions[tr.row0];
    const int lo_t = first_visible(a, pos0), hi_t = pos0 + tr.ntok - 1;     // the keys that some row of the tile sees
    const int* table = a.block_tables + static_cast<size_t>(a.row_req[tr.row0]) * a.table_stride;
    const bf* kc = static_cast<const bf*>(a.k_cache);
    const bf* vc = static_cast<const bf*>(a.v_cache);
    const int k_chunks = a.hd / 8, v_chunks = a.vd / 8;
    const int all_tiles = (hi_t - lo_t) / kRowsTile + 1;
    const int per_split = (all_tiles + rt.splits - 1) / rt.splits;
    const int it0 = split * per_split, it1 = min(all_tiles, it0 + per_split);

    // lane j looks up the page row of key j of a tile: one load in flight per lane instead of a chain of dependent ones;
    // the rows of the tile after the next are asked for before the current tile's products, a tile ahead of their use
    auto lookup = [&](int tile) -> long long {
        const int pl = lo_t + tile * kRowsTile + lane;
        if (tile >= it1 || pl > hi_t) return -1;
        return (static_cast<long long>(table[pl / a.page_size]) * a.Hkv + g) * a.page_size + (pl % a.page_size);
    };
    auto fetch = [&](long long my_row, int stage) {
        for (int j = warp; j < kRowsTile; j += 4) {
            const long long rj = __shfl_sync(0xffffffffu, my_row, j);
            const bool in = rj >= 0;
            const size_t row = in ? static_cast<size_t>(rj) : 0;
            const bf* src = kc + row * a.hd;
            const uint32_t dst = rows_smem_u32(s_k + (stage * kRowsTile + j) * qs);
            for (int c = lane; c < k_chunks; c += 32) rows_cp_async16(dst + c * 16, src + c * 8, in ? 16 : 0);   // 0 bytes: zeros
            if (!a.alias) {
                const bf* vsrc = vc + row * a.v_row;
                const uint32_t vdst = rows_smem_u32(s_v + (stage * kRowsTile + j) * vs);
                for (int c = lane; c < v_chunks; c += 32) rows_cp_async16(vdst + c * 16, vsrc + c * 8, in ? 16 : 0);
            }
        }
        rows_cp_async_commit();
    };

    if (it0 < it1) fetch(lookup(it0), 0);
    long long next_rows = lookup(it0 + 1);
    // the queries, a warp per row: 16-byte loads where the rows allow them
    for (int r = warp; r < RT; r += 4) {
        bf* dst = s_q + r * qs;
        if (!row_on(r)) {
            for (int d = lane; d < a.hd; d += 32) dst[d] = __float2bfloat16_rn(0.f);
            continue;
        }
        const size_t off = static_cast<size_t>(tr.row0 + tr.token(r)) * a.ldq + static_cast<size_t>(g * group + first_head + tr.head(r)) * a.hd;
        if (a.q_is_f32) {
            const float* src = static_cast<const float*>(a.q) + off;
            if (a.ldq % 4 == 0 && reinterpret_cast<uintptr_t>(a.q) % 16 == 0) {
                for (int d = lane * 4; d < a.hd; d += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(src + d);
                    *reinterpret_cast<uint2*>(dst + d) = make_uint2(rows_pack(v.x, v.y), rows_pack(v.z, v.w));
                }
            } else {
                for (int d = lane; d < a.hd; d += 32) dst[d] = __float2bfloat16_rn(src[d]);
            }
        } else {
            const bf* src = static_cast<const bf*>(a.q) + off;
            if (a.ldq % 8 == 0 && reinterpret_cast<uintptr_t>(a.q) % 16 == 0) {
                for (int d = lane * 8; d < a.hd; d += 256) *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(src + d);
            } else {
                for (int d = lane; d < a.hd; d += 32) dst[d] = src[d];
            }
        }
    }

    const int gr = lane >> 2, tq = lane & 3;            // the fragment's rows gr and gr + 8 and its pair of columns
    const int rb = OWN ? warp * kMmaHeads : PAIR ? (warp >> 1) * kMmaHeads : 0;      // the first of this warp's sixteen rows
    float o[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, slope[2] = {0.f, 0.f};
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = rb + gr + 8 * h;
        const bool on = row_on(r);
        pos_r[h] = on ? pos0 + tr.token(r) : -1;                  // a row that is not there sees no key
        lo_r[h] = on ? first_visible(a, pos_r[h]) : 0;
        if (a.slopes && on) slope[h] = a.slopes[g * group + first_head + tr.head(r)];
    }
    const int nv = OWN ? a.vd / 8 : PAIR ? a.vd / 16 : a.vd / 32;                     // 8-wide value tiles of this warp
    const int v0 = OWN ? 0 : PAIR ? (warp & 1) * (a.vd / 2) : warp * (a.vd / 4);      // its first value dimension
    const bool warp_on = OWN ? rb < n_rows : PAIR ? (warp >> 1) < tr.ntok : true;    // (a warp without rows only helps to fetch)
    const int k_steps = a.hd / 16;

    for (int it = it0; it < it1; ++it) {
        const int st = (it - it0) & 1;
        rows_cp_async_wait_all();
        __syncthreads();                                 // tile ``it`` is there; everyone is done with the other stage
        if (it + 1 < it1) fetch(next_rows, st ^ 1);
        next_rows = lookup(it + 2);
        const bf* kt = s_k + st * kRowsTile * qs;
        const bf* vt = s_v + st * kRowsTile * vs;
        // S = Q K^T, this warp's slices of the head dimension
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
        const uint32_t q_addr = rows_smem_u32(s_q + (rb + (lane & 15)) * qs + (lane >> 4) * 8);
        const uint32_t k_addr = rows_smem_u32(kt + ((lane >> 4) * 8 + (lane & 7)) * qs + ((lane >> 3) & 1) * 8);
        if (warp_on) {
            for (int ks = MODE ? 0 : warp; ks < k_steps; ks += MODE ? 1 : 4) {
                uint32_t qa[4];
                rows_ldsm_x4(q_addr + ks * 32, qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t b0, b1, b2, b3;
                    rows_ldsm_x4(k_addr + half * 16 * qs * 2 + ks * 32, b0, b1, b2, b3);
                    rows_mma(s[half * 2], qa, b0, b1);
                    rows_mma(s[half * 2 + 1], qa, b2, b3);
                }
            }
        }
        if (MODE == 0) {
            float* mine = s_s + warp * kMmaHeads * kMmaSStride;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                *reinterpret_cast<float2*>(mine + gr * kMmaSStride + nt * 8 + 2 * tq) = make_float2(s[nt][0], s[nt][1]);
                *reinterpret_cast<float2*>(mine + (gr + 8) * kMmaSStride + nt * 8 + 2 * tq) = make_float2(s[nt][2], s[nt][3]);
            }
            __syncthreads();
        }
        if (!warp_on) continue;
        // every warp adds the four partial sums in warp order and takes the softmax step of all sixteen rows
        const int base = lo_t + it * kRowsTile;
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            if (MODE == 0) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float2 part = *reinterpret_cast<const float2*>(s_s + (w * kMmaHeads + gr + 8 * h) * kMmaSStride + nt * 8 + 2 * tq);
                        sum2.x += part.x; sum2.y += part.y;
                    }
                    s[nt][2 * h] = sum2.x; s[nt][2 * h + 1] = sum2.y;
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1, col = nt * 8 + 2 * tq + (e & 1);
                float v = s[nt][e];
                const int key = base + col;
                v = (key >= lo_r[h] && key <= pos_r[h]) ? capped(v * a.scale, a.softcap) - slope[h] * static_cast<float>(pos_r[h] - key) : -INFINITY;
                s[nt][e] = v;
                tile_max[h] = fmaxf(tile_max[h], v);
            }
        }
        float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
            tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
            const float m_new = fmaxf(m[h], tile_max[h]);            // -inf while the row has seen no key yet
            corr[h] = m[h] == -INFINITY ? 0.f : expf(m[h] - m_new);
            m[h] = m_new;
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = s[nt][e] == -INFINITY ? 0.f : expf(s[nt][e] - m[e >> 1]);
                s[nt][e] = p;
                sum[e >> 1] += p;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
            sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
            l[h] = l[h] * corr[h] + sum[h];
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        // O += P V, this warp's quarter of the value dimensions
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t pa[4] = {rows_pack(s[2 * ks][0], s[2 * ks][1]), rows_pack(s[2 * ks][2], s[2 * ks][3]),
                              rows_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), rows_pack(s[2 * ks + 1][2], s[2 * ks + 1][3])};
            const uint32_t v_addr = rows_smem_u32(vt + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * vs + v0 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < NV / 2; ++np) {
                if (2 * np < nv) {
                    uint32_t b0, b1, b2, b3;
                    rows_ldsm_x4_trans(v_addr + np * 32, b0, b1, b2, b3);
                    rows_mma(o[2 * np], pa, b0, b1);
                    rows_mma(o[2 * np + 1], pa, b2, b3);
                }
            }
        }
    }
    rows_cp_async_wait_all();

    if (rt.splits > 1) {
        // this range's unnormalised sums, maximum and weight: merged by attention_rows_merge_kernel
        float* ws = rt.workspace + ((((static_cast<size_t>(blockIdx.x) * a.Hkv + g) * rt.head_blocks + zb) * rt.splits + split) * RT) * (a.vd + 2);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float* row = ws + static_cast<size_t>(rb + gr + 8 * h) * (a.vd + 2);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (i < nv) { row[v0 + i * 8 + 2 * tq] = o[i][2 * h]; row[v0 + i * 8 + 2 * tq + 1] = o[i][2 * h + 1]; }
            }
            if ((OWN || (PAIR && !(warp & 1)) || warp == 0) && tq == 0) { row[a.vd] = m[h]; row[a.vd + 1] = l[h]; }
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = rb + gr + 8 * h;
        if (!row_on(r)) continue;
        const int head = g * group + first_head + tr.head(r);
        float M = m[h], L = l[h], f = 1.f;
        if (a.sinks) {
            const float sk = a.sinks[head];
            M = fmaxf(M, sk);
            f = expf(m[h] - M);
            L = L * f + expf(sk - M);
        }
        const float mul = f / L;
        const size_t ob = static_cast<size_t>(tr.row0 + tr.token(r)) * a.ldo + static_cast<size_t>(head) * a.vd + v0 + 2 * tq;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nv) {
                const float x0 = o[i][2 * h] * mul, x1 = o[i][2 * h + 1] * mul;
                if (a.out_is_f32) *reinterpret_cast<float2*>(static_cast<float*>(a.out) + ob + i * 8) = make_float2(x0, x1);
                else *reinterpret_cast<uint32_t*>(static_cast<bf*>(a.out) + ob + i * 8) = rows_pack(x0, x1);
            }
        }
    }
}

// Merges the ranges of keys of a tile, in their order: one block per (tile, key/value head and block of heads, row).
__global__ void __launch_bounds__(128)
attention_rows_merge_kernel(const RowsArgs a, const RowTiles rt) {
    pdl_prologue();
    __shared__ float s_w[16];
    __shared__ float s_inv;
    const int g = blockIdx.y / rt.head_blocks, zb = blockIdx.y % rt.head_blocks, r = blockIdx.z;
    const int group = a.H / a.Hkv;
    const TileRows tr = tile_rows(rt, blockIdx.x, group);
    const int first_head = zb * kMmaHeads;
    const int n_heads = min(kMmaHeads, group - first_head);
    const bool on = rt.block_rows == 2 * kMmaHeads ? ((r >> 4) < tr.ntok && (r & 15) < n_heads)
                  : (rt.block_rows == kMmaHeads && tr.gp == kMmaHeads) ? r < n_heads : r < tr.ntok * tr.gp;
    if (!on) return;
    const size_t stride = static_cast<size_t>(rt.block_rows) * (a.vd + 2);
    const float* row = rt.workspace + (((static_cast<size_t>(blockIdx.x) * a.Hkv + g) * rt.head_blocks + zb) * rt.splits) * stride +
                       static_cast<size_t>(r) * (a.vd + 2);
    const int head = g * group + first_head + tr.head(r);
    if (threadIdx.x < 32) {
        const int s = threadIdx.x;
        const float ms = s < rt.splits ? row[s * stride + a.vd] : -INFINITY;
        const float ls = s < rt.splits ? row[s * stride + a.vd + 1] : 0.f;
        float M = warp_max(ms);
        if (a.sinks) M = fmaxf(M, a.sinks[head]);
        const float w = ms == -INFINITY ? 0.f : expf(ms - M);
        float L = 0.f;
        for (int i = 0; i < rt.splits; ++i) L += __shfl_sync(0xffffffffu, ls * w, i);       // in the ranges' order
        if (a.sinks) L += expf(a.sinks[head] - M);
        if (s < 16) s_w[s] = w;
        if (s == 0) s_inv = 1.0f / L;
    }
    __syncthreads();
    const size_t ob = static_cast<size_t>(tr.row0 + tr.token(r)) * a.ldo + static_cast<size_t>(head) * a.vd;
    for (int d = threadIdx.x; d < a.vd; d += 128) {
        float v = 0.f;
#pragma unroll 4
        for (int s = 0; s < rt.splits; ++s) v = fmaf(row[s * stride + d], s_w[s], v);
        v *= s_inv;
        if (a.out_is_f32) static_cast<float*>(a.out)[ob + d] = v;
        else static_cast<__nv_bfloat16*>(a.out)[ob + d] = __float2bfloat16_rn(v);
    }
}

template <int NV, int MODE>
static int launch_rows_mma(const RowsArgs& a, const RowTiles& rt, int n_tiles, size_t smem, cudaStream_t st) {
    auto kernel = attention_rows_mma_kernel<NV, MODE>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { set_error("attention_rows: %s", cudaGetErrorString(e)); return 1; }
    }
    launch_kernel(kernel, dim3(n_tiles, a.Hkv, rt.head_blocks * rt.splits), dim3(128), smem, st, a, rt);
    if (check_launch("attention_rows (tensor cores)")) return 1;
    if (rt.splits > 1) {
        launch_kernel(attention_rows_merge_kernel, dim3(n_tiles, a.Hkv * rt.head_blocks, rt.block_rows), dim3(128), 0, st, a, rt);
        return check_launch("attention_rows (merge)");
    }
    return 0;
}

constexpr int kRowsMaxValueDim = 512;
constexpr int kRowsMaxHeadDim = 1024;

template <typename T, int HPW, int VI>
static int launch_rows(const RowsArgs& a, int T_rows, int blocks_z, int warps, size_t smem, cudaStream_t st) {
    auto kernel = attention_rows_kernel<T, HPW, VI>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { set_error("attention_rows: %s", cudaGetErrorString(e)); return 1; }
    }
    launch_kernel(kernel, dim3(T_rows, a.Hkv, blocks_z), dim3(warps * 32), smem, st, a);
    return check_launch("attention_rows");
}

template <typename T, int HPW>
static int launch_rows_vi(const RowsArgs& a, int T_rows, int blocks_z, int warps, size_t smem, cudaStream_t st) {
    if (a.vd <= 128) return launch_rows<T, HPW, 4>(a, T_rows, blocks_z, warps, smem, st);
    if (a.vd <= 256) return launch_rows<T, HPW, 8>(a, T_rows, blocks_z, warps, smem, st);
    return launch_rows<T, HPW, 16>(a, T_rows, blocks_z, warps, smem, st);
}

}  // namespace gi

using namespace gi;

static int g_rows_mma = 1;
static int g_rows_pairs = 1;
// 0: large heads run with the four warps sharing a token's sixteen rows instead of two tokens a block (for comparisons)
extern "C" int gi_attention_rows_set_pairs(int on) { const int old = g_rows_pairs; g_rows_pairs = on ? 1 : 0; return old; }
// 0: the CUDA-core form also where the tensor-core form applies (for comparisons); returns the old setting
extern "C" int gi_attention_rows_set_mma(int on) { const int old = g_rows_mma; g_rows_mma = on ? 1 : 0; return old; }

extern "C" int gi_attention_rows_supported(int hd, int vd) {
    return hd >= 1 && hd <= kRowsMaxHeadDim && vd >= 1 && vd <= kRowsMaxValueDim;
}

// Whether every warp owns sixteen rows of a block of 64 (small heads) instead of the four warps sharing sixteen.
static bool rows_mma_own(int group, int hd, int vd) { return hd <= 128 && vd <= 128 && group <= kMmaHeads; }

static size_t rows_mma_smem_of(int mode, int hd, int vd, bool alias) {
    const int qs = hd + kMmaPad, vs = vd + kMmaPad;
    const int rows = mode == 1 ? kMmaOwnRows : mode == 2 ? 2 * kMmaHeads : kMmaHeads;
    return static_cast<size_t>(rows + 2 * kRowsTile) * qs * 2 + (alias ? 0 : static_cast<size_t>(2 * kRowsTile) * vs * 2) +
           (mode == 0 ? static_cast<size_t>(4 * kMmaHeads * kMmaSStride) * 4 : 0);
}

// 0: the warps share sixteen rows; 1: a warp owns sixteen of 64 rows; 2: two tokens of sixteen heads, two warps a token.
static int rows_mma_mode(int group, int hd, int vd, bool alias) {
    if (rows_mma_own(group, hd, vd)) return 1;
    if (g_rows_pairs && group >= kMmaHeads && rows_mma_smem_of(2, hd, vd, alias) <= 113 * 1024) return 2;      // two blocks an SM
    return 0;
}

static size_t rows_mma_smem(int group, int hd, int vd, bool alias) { return rows_mma_smem_of(rows_mma_mode(group, hd, vd, alias), hd, vd, alias); }

// How many consecutive tokens of one request share a tile of the tensor-core form (16 / group, at least 1), or 0 when
// that form does not serve these sizes (a bfloat16 cache is understood): the head size in whole 16s, the value size
// in whole 64s up to 512.
extern "C" int gi_attention_rows_tile_tokens(int H, int Hkv, int hd, int vd, int values_in_keys) {
    if (!g_rows_mma || Hkv <= 0 || H % Hkv || hd % 16 || vd % 64 || vd > kRowsMaxValueDim || hd > kRowsMaxHeadDim) return 0;
    const int group = H / Hkv;
    if (rows_mma_smem(group, hd, vd, values_in_keys != 0) > 200 * 1024) return 0;
    const int mode = rows_mma_mode(group, hd, vd, values_in_keys != 0);
    if (mode == 1) return kMmaOwnRows / group;
    if (mode == 2) return 2;
    return group >= kMmaHeads ? 1 : kMmaHeads / group;
}

static int gi_attention_rows_impl(const void* q, int q_dtype, int ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                                 void* out, int out_dtype, int ldo, const int* row_req, const int* positions,
                                 const int* block_tables, int table_stride, int T, int H, int Hkv, int hd, int vd, int v_row,
                                 int values_in_keys, int page_size, float scale, float softcap, int window, int chunk, const float* slopes,
                                 const float* sinks, const int* tile_list, int list_kind, int n_tiles, int splits, float* workspace,
                                 long long workspace_floats, void* stream) {
    if (T == 0 || (list_kind != 0 && n_tiles == 0)) return 0;
    GI_REQUIRE(T > 0 && H > 0 && Hkv > 0 && page_size > 0, "attention_rows: sizes must be positive");
    GI_REQUIRE(H % Hkv == 0, "attention_rows: %d query heads are not a multiple of %d key/value heads", H, Hkv);
    GI_REQUIRE(gi_attention_rows_supported(hd, vd), "attention_rows: head size %d / value size %d is not supported (up to %d / %d)",
               hd, vd, kRowsMaxHeadDim, kRowsMaxValueDim);
    GI_REQUIRE(!values_in_keys || (vd <= hd && v_row == hd), "attention_rows: values inside the key rows must fit them");
    GI_REQUIRE(v_row >= vd && ldq >= H * hd && ldo >= H * vd, "attention_rows: a row is shorter than its heads");
    GI_REQUIRE(Hkv <= 65535, "attention_rows: too many key/value heads for one launch");
    GI_REQUIRE((q_dtype == kF32 || q_dtype == kBF16) && (out_dtype == kF32 || out_dtype == kBF16) &&
               (cache_dtype == kF32 || cache_dtype == kBF16), "attention_rows: unsupported dtype code");
    const int group = H / Hkv;
    RowsArgs a;
    a.q = q; a.q_is_f32 = q_dtype == kF32; a.ldq = ldq;
    a.k_cache = k_cache; a.v_cache = values_in_keys ? k_cache : v_cache;
    a.out = out; a.out_is_f32 = out_dtype == kF32; a.ldo = ldo;
    a.row_req = row_req; a.positions = positions; a.block_tables = block_tables; a.table_stride = table_stride;
    a.H = H; a.Hkv = Hkv; a.hd = hd; a.vd = vd; a.v_row = v_row; a.page_size = page_size;
    a.scale = scale; a.softcap = softcap; a.window = window; a.chunk = chunk; a.slopes = slopes; a.sinks = sinks;
    a.alias = values_in_keys ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // bfloat16 cache and sizes in whole MMA tiles: the tensor-core form (tiles of rows from the caller's list, or a row each)
    const int tile_tokens = cache_dtype == kBF16 && ldo % 2 == 0 ? gi_attention_rows_tile_tokens(H, Hkv, hd, vd, values_in_keys) : 0;
    GI_REQUIRE(list_kind == 0 || tile_tokens > 0, "attention_rows: lists of tiles are for the tensor-core form, which does not serve these sizes");
    if (tile_tokens > 0 && (list_kind != 0 || group >= 8)) {
        RowTiles rt;
        rt.list = tile_list; rt.kind = list_kind;
        rt.head_blocks = (group + kMmaHeads - 1) / kMmaHeads;
        rt.splits = splits > 1 ? splits : 1;
        int mode = rows_mma_mode(group, hd, vd, a.alias != 0);
        if (mode == 2 && list_kind != 2) mode = 0;        // single tokens: all four warps on the one token
        rt.block_rows = mode == 1 ? kMmaOwnRows : mode == 2 ? 2 * kMmaHeads : kMmaHeads;
        rt.workspace = workspace;
        const int tiles = list_kind == 0 ? T : n_tiles;
        GI_REQUIRE(list_kind == 0 || tile_list != nullptr, "attention_rows: the list of tiles is missing");
        GI_REQUIRE(rt.splits == 1 || (workspace != nullptr && static_cast<long long>(tiles) * Hkv * rt.head_blocks * rt.splits * rt.block_rows * (vd + 2) <= workspace_floats),
                   "attention_rows: the workspace of the key ranges is missing or too small");
        GI_REQUIRE(rt.head_blocks * rt.splits <= 65535 && a.Hkv * rt.head_blocks <= 65535 && rt.splits <= 16,
                   "attention_rows: too many blocks of heads or ranges of keys (at most 16 ranges)");
        const size_t smem_mma = rows_mma_smem_of(mode, hd, vd, a.alias != 0);
        if (mode == 1) return vd <= 64 ? launch_rows_mma<8, 1>(a, rt, tiles, smem_mma, st) : launch_rows_mma<16, 1>(a, rt, tiles, smem_mma, st);
        if (mode == 2) return vd <= 256 ? launch_rows_mma<16, 2>(a, rt, tiles, smem_mma, st) : launch_rows_mma<32, 2>(a, rt, tiles, smem_mma, st);
        if (vd <= 128) return launch_rows_mma<4, 0>(a, rt, tiles, smem_mma, st);
        if (vd <= 256) return launch_rows_mma<8, 0>(a, rt, tiles, smem_mma, st);
        return launch_rows_mma<16, 0>(a, rt, tiles, smem_mma, st);
    }
    // rows of the key tile: pairs of values are read by 32 lanes from 32 rows, free of bank conflicts when the row
    // length counted in pairs is odd
    const int hdp = (hd + 1) & ~1;
    a.ks = (hdp / 2) % 2 ? hdp : hdp + 2;
    // few heads in a group: a warp per head; many: four heads per warp, up to sixteen per block
    const int hpw = group <= 4 ? 1 : 4;
    a.heads_per_block = group <= 4 ? group : std::min((group + 3) / 4 * 4, 16);
    const int warps = a.heads_per_block / hpw;
    const int blocks_z = (group + a.heads_per_block - 1) / a.heads_per_block;
    const size_t esz = cache_dtype == kF32 ? 4 : 2;
    const size_t smem = static_cast<size_t>(a.heads_per_block) * hdp * 4 + static_cast<size_t>(kRowsTile) * a.ks * esz +
                        (a.alias ? 0 : static_cast<size_t>(kRowsTile) * vd * esz);
    GI_REQUIRE(smem <= 200 * 1024, "attention_rows: head size %d with %d heads per block needs %zu bytes of shared memory", hd,
               a.heads_per_block, smem);
    if (cache_dtype == kF32)
        return hpw == 1 ? launch_rows_vi<float, 1>(a, T, blocks_z, warps, smem, st) : launch_rows_vi<float, 4>(a, T, blocks_z, warps, smem, st);
    return hpw == 1 ? launch_rows_vi<__nv_bfloat16, 1>(a, T, blocks_z, warps, smem, st)
                    : launch_rows_vi<__nv_bfloat16, 4>(a, T, blocks_z, warps, smem, st);
}

extern "C" int gi_attention_rows(const void* q, int q_dtype, int ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                                 void* out, int out_dtype, int ldo, const int* row_req, const int* positions,
                                 const int* block_tables, int table_stride, int T, int H, int Hkv, int hd, int vd, int v_row,
                                 int values_in_keys, int page_size, float scale, float softcap, int window, int chunk, const float* slopes,
                                 const float* sinks, const int* tile_list, int list_kind, int n_tiles, int splits, float* workspace,
                                 long long workspace_floats, void* stream) {
    return gi::dispatch(gi_attention_rows_impl, q, q_dtype, ldq, k_cache, v_cache, cache_dtype, out, out_dtype, ldo, row_req,
                        positions, block_tables, table_stride, T, H, Hkv, hd, vd, v_row, values_in_keys, page_size, scale, softcap, window,
                        chunk, slopes, sinks, tile_list, list_kind, n_tiles, splits, workspace, workspace_floats, stream);
}
