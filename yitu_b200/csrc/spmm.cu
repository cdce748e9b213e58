// CSR pull SpMM for sm_100a:  out[r,:] = act(alpha*row_scale[r] * sum_{e in row r} w(e) * x[col_e,:] + bias)
//
// Work decomposition
//   * a group of LPR lanes (4..32, one warp for rows of >= 128 floats) owns one destination row, or one
//     chunk of a hub row; each lane keeps NV independent 128-bit accumulators, so a warp has up to
//     4 edges x NV x 512 B of feature gathers in flight;
//   * column ids / edge weights are fetched LPR at a time, one per lane (coalesced, streamed past L1)
//     and broadcast with warp shuffles, so the gather loop issues nothing but 128-bit loads and FMAs;
//   * rows longer than plan->chunk_edges are cut into chunks handled by the first n_chunks groups of the
//     grid (scheduled first: they are the longest tasks); partial sums land in scratch and a second tiny
//     kernel adds them in chunk order.  No float atomics anywhere: results are run-to-run identical.
//
// Measured alternatives that lost on B200 and are not kept: staging rows in a shared-memory ring with
// cp.async.bulk + mbarrier (2.2x slower: 1 KiB per bulk copy is too fine a grain) or per-lane cp.async (equal
// at best, only at the same occupancy); sub-warp groups narrower than the row (lose coalescing); a persistent
// grid with software-pipelined row pointers / index tiles (1.7x slower than letting the CTA scheduler
// balance short CTAs); batches of 8 consecutive rows per warp with the next row's index tile prefetched
// (1.1-1.4x slower: fewer, longer warps hide less latency than many short ones); for heads that share one source
// row (x_shared_heads), a lane-per-feature layout with the H edge weights broadcast by shuffle (5.4 ms against 3.7 ms
// for the per-head layout below on the 8x32 layer: ten shuffles per edge cost more than the replicated loads).
//
// The kernel is bound by HBM/L2 gather bandwidth; algorithmic bytes per edge = 4*D + 4 (+4 with edge
// values), per row = 4*D written + one row pointer.

#include <cstdlib>

#include "common.cuh"

namespace yitu {

struct SpmmParams {
    int64_t n_rows, n_cols, D, H, F;
    const void *indptr;
    const int *indices;
    int is64, mask, wmode, accumulate;
    const float *values;
    const int *perm;
    const float *norm_dst, *norm_src, *row_scale;
    float alpha;
    const float *x;
    int64_t xs;
    float *out;
    int64_t os;
    int64_t n_chunks;     // chunks of the hub schedule (> 0: rows longer than chunk_edges are not aggregated as rows)
    int64_t chunk_tasks;  // how many of them THIS launch aggregates (its first groups): n_chunks, or 0
    int64_t row_tasks;    // rows THIS launch aggregates: n_rows, or 0 for a launch that takes the chunks only
    int chunk_edges;
    const int *chunk_row;
    const int64_t *chunk_begin;
    float *scratch;
    const float *bias;
    int act, xshared;
};

// Last step of every output row: bias, then activation (both optional).
template <int VEC>
__device__ __forceinline__ void finish_vec(float (&r)[VEC], const SpmmParams &p, int64_t d) {
    if (p.bias) {
#pragma unroll
        for (int q = 0; q < VEC; ++q) r[q] += __ldg(p.bias + d + q);
    }
    if (p.act) {
#pragma unroll
        for (int q = 0; q < VEC; ++q) r[q] = activate(r[q], p.act);
    }
}

template <int LPR, int NV, int VEC, int EU, bool PER_HEAD, bool IDX32>
__global__ void __launch_bounds__(256) spmm_kernel(const __grid_constant__ SpmmParams p) {
    static_assert(EU <= LPR && (EU & (EU - 1)) == 0, "edge unroll must be a power of two <= lanes per row");
    const int lane = threadIdx.x & 31;
    const int l = lane & (LPR - 1);
    const unsigned gmask = (LPR == 32) ? 0xffffffffu : (((1u << LPR) - 1u) << (lane & ~(LPR - 1)));
    const int64_t gid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / LPR;
    const int64_t d0 = static_cast<int64_t>(blockIdx.y) * (LPR * NV * VEC);

    int64_t row, eb, ee;
    float *dst;
    bool raw;
    if (gid < p.chunk_tasks) {
        row = __ldg(p.chunk_row + gid);
        eb = __ldg(p.chunk_begin + gid);
        const int64_t rend = load_ptr(p.indptr, p.is64, row + 1);
        ee = min(eb + static_cast<int64_t>(p.chunk_edges), rend);
        dst = p.scratch + gid * p.D;
        raw = true;
    } else {
        row = gid - p.chunk_tasks;
        if (row >= p.row_tasks) return;
        eb = load_ptr(p.indptr, p.is64, row);
        ee = load_ptr(p.indptr, p.is64, row + 1);
        if (p.n_chunks > 0 && ee - eb > p.chunk_edges) return;  // hub row: done by its chunks
        dst = p.out + row * p.os;
        raw = false;
    }

    int64_t off[NV];
    bool valid[NV];
    int hd[NV];
    int64_t xo[NV];  // offset of the lane's slice inside a source row (differs from off[] when heads share x)
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        off[i] = d0 + static_cast<int64_t>(i * LPR + l) * VEC;
        valid[i] = off[i] < p.D;
        hd[i] = PER_HEAD ? static_cast<int>(off[i] / p.F) : 0;
        xo[i] = (PER_HEAD && p.xshared) ? off[i] - static_cast<int64_t>(hd[i]) * p.F : off[i];
    }

    float acc[NV][VEC];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[i][v] = 0.0f;

    const float nd = (p.wmode == YITU_W_NODE) ? __ldg(p.norm_dst + row) : 0.0f;

    for (int64_t e0 = eb; e0 < ee; e0 += LPR) {
        const int n = static_cast<int>(min(static_cast<int64_t>(LPR), ee - e0));
        int my_col = 0, my_vi = 0;
        float my_w = 0.0f;
        if (l < n) {
            const int64_t e = e0 + l;
            const int rawidx = ld_stream(p.indices + e);
            my_col = p.mask ? (rawidx & p.mask) : rawidx;
            if constexpr (PER_HEAD) {
                my_vi = p.perm ? ld_stream(p.perm + e) : static_cast<int>(e);
            } else {
                if (p.wmode == YITU_W_NONE) {
                    my_w = 1.0f;
                } else if (p.wmode == YITU_W_NODE) {
                    my_w = nd * __ldg(p.norm_src + my_col);
                } else {
                    const int64_t vi = p.perm ? static_cast<int64_t>(ld_stream(p.perm + e)) : e;
                    my_w = ld_stream(p.values + vi);
                }
            }
        }
        // lanes past the end of the row repeat the tile's first edge with weight 0, so the gather loop
        // below runs in steps of EU edges without a remainder path (the repeated row is an L1 hit)
        const int c_first = __shfl_sync(gmask, my_col, 0, LPR);
        const int v_first = PER_HEAD ? __shfl_sync(gmask, my_vi, 0, LPR) : 0;
        if (l >= n) {
            my_col = c_first;
            my_vi = v_first;
        }
        const int n_up = (n + EU - 1) & ~(EU - 1);
        for (int j = 0; j < n_up; j += EU) {
            int c[EU], vi[EU];
            float w[EU];
#pragma unroll
            for (int u = 0; u < EU; ++u) {
                c[u] = __shfl_sync(gmask, my_col, j + u, LPR);
                if constexpr (PER_HEAD) {
                    vi[u] = __shfl_sync(gmask, my_vi, j + u, LPR);
                } else {
                    w[u] = __shfl_sync(gmask, my_w, j + u, LPR);
                }
            }
            float v[EU][NV][VEC];
            float wh[EU][NV];
#pragma unroll
            for (int u = 0; u < EU; ++u) {
                const float *xr = p.x + static_cast<int64_t>(c[u]) * p.xs;
                // 32-bit element offsets when the feature matrix has fewer than 2^32 elements
                const uint32_t xr32 = static_cast<uint32_t>(c[u]) * static_cast<uint32_t>(p.xs);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (valid[i]) {
                        if constexpr (IDX32) load_vec<VEC>(v[u][i], p.x + (xr32 + static_cast<uint32_t>(xo[i])));
                        else load_vec<VEC>(v[u][i], xr + xo[i]);
                        if constexpr (PER_HEAD)
                            wh[u][i] = (j + u < n) ? __ldg(p.values + static_cast<int64_t>(vi[u]) * p.H + hd[i]) : 0.0f;
                    } else {
#pragma unroll
                        for (int q = 0; q < VEC; ++q) v[u][i][q] = 0.0f;
                        wh[u][i] = 0.0f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < EU; ++u)
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const float ww = PER_HEAD ? wh[u][i] : w[u];
#pragma unroll
                    for (int q = 0; q < VEC; ++q) acc[i][q] = fmaf(ww, v[u][i][q], acc[i][q]);
                }
        }
    }

    if (raw) {
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (valid[i]) store_vec<VEC>(dst + off[i], acc[i]);
    } else {
        const float s = p.alpha * (p.row_scale ? __ldg(p.row_scale + row) : 1.0f);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (!valid[i]) continue;
            float r[VEC];
            if (p.accumulate) {
                load_vec<VEC>(r, dst + off[i]);
#pragma unroll
                for (int q = 0; q < VEC; ++q) r[q] = fmaf(s, acc[i][q], r[q]);
            } else {
#pragma unroll
                for (int q = 0; q < VEC; ++q) r[q] = s * acc[i][q];
            }
            finish_vec<VEC>(r, p, off[i]);
            store_vec<VEC>(dst + off[i], r);
        }
    }
}

// Rows of at most 128 floats with 256-bit loads: the warp still owns one destination row (or hub chunk), but one
// load instruction now fetches 32 / LPE edges at once — LPE = D/8 lanes (32 bytes each) cover a source row, so the
// lanes of sub-group s gather edge s of every step.  Each sub-group accumulates its own edges; a butterfly over the
// sub-groups adds them up at the end of the row.  Scalar weights only (no per-head values).
template <int LPE, int EU, bool IDX32>
__global__ void __launch_bounds__(256) spmm_wide_kernel(const __grid_constant__ SpmmParams p) {
    constexpr int EPI = 32 / LPE;  // edges per load instruction
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPE, l = lane & (LPE - 1);
    const int64_t gid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    int64_t row, eb, ee;
    float *dst;
    bool raw;
    if (gid < p.chunk_tasks) {
        row = __ldg(p.chunk_row + gid);
        eb = __ldg(p.chunk_begin + gid);
        const int64_t rend = load_ptr(p.indptr, p.is64, row + 1);
        ee = min(eb + static_cast<int64_t>(p.chunk_edges), rend);
        dst = p.scratch + gid * p.D;
        raw = true;
    } else {
        row = gid - p.chunk_tasks;
        if (row >= p.row_tasks) return;
        eb = load_ptr(p.indptr, p.is64, row);
        ee = load_ptr(p.indptr, p.is64, row + 1);
        if (p.n_chunks > 0 && ee - eb > p.chunk_edges) return;
        dst = p.out + row * p.os;
        raw = false;
    }
    const int off = l * 8;
    const bool valid = off < p.D;
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
    const float nd = (p.wmode == YITU_W_NODE) ? __ldg(p.norm_dst + row) : 0.0f;

    for (int64_t e0 = eb; e0 < ee; e0 += 32) {
        const int n = static_cast<int>(min(static_cast<int64_t>(32), ee - e0));
        int my_col = 0;
        float my_w = 0.0f;
        if (lane < n) {
            const int64_t e = e0 + lane;
            const int rawidx = ld_stream(p.indices + e);
            my_col = p.mask ? (rawidx & p.mask) : rawidx;
            if (p.wmode == YITU_W_NONE) {
                my_w = 1.0f;
            } else if (p.wmode == YITU_W_NODE) {
                my_w = nd * __ldg(p.norm_src + my_col);
            } else {
                const int64_t vi = p.perm ? static_cast<int64_t>(ld_stream(p.perm + e)) : e;
                my_w = ld_stream(p.values + vi);
            }
        }
        const int c_first = __shfl_sync(0xffffffffu, my_col, 0);
        if (lane >= n) my_col = c_first;  // weight 0, a row that is in flight anyway
        constexpr int STEP = EPI * EU;     // edges per unrolled step
        const int n_up = (n + STEP - 1) / STEP * STEP;
        for (int j = 0; j < n_up; j += STEP) {
            int c[EU];
            float w[EU];
#pragma unroll
            for (int u = 0; u < EU; ++u) {
                const int idx = (j + u * EPI + sub) & 31;
                c[u] = __shfl_sync(0xffffffffu, my_col, idx);
                w[u] = (j + u * EPI + sub < 32) ? __shfl_sync(0xffffffffu, my_w, idx) : (__shfl_sync(0xffffffffu, my_w, idx), 0.0f);
            }
            float v[EU][8];
#pragma unroll
            for (int u = 0; u < EU; ++u) {
                if (valid) {
                    if constexpr (IDX32)
                        load_vec<8>(v[u], p.x + (static_cast<uint32_t>(c[u]) * static_cast<uint32_t>(p.xs) + static_cast<uint32_t>(off)));
                    else
                        load_vec<8>(v[u], p.x + static_cast<int64_t>(c[u]) * p.xs + off);
                } else {
#pragma unroll
                    for (int q = 0; q < 8; ++q) v[u][q] = 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < EU; ++u)
#pragma unroll
                for (int q = 0; q < 8; ++q) acc[q] = fmaf(w[u], v[u][q], acc[q]);
        }
    }
    // add the sub-groups' partial sums (fixed order: deterministic)
#pragma unroll
    for (int o = LPE; o < 32; o <<= 1)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], o);
    if (sub != 0 || !valid) return;
    if (raw) {
        store_vec<8>(dst + off, acc);
    } else {
        const float s = p.alpha * (p.row_scale ? __ldg(p.row_scale + row) : 1.0f);
        float r[8];
        if (p.accumulate) {
            load_vec<8>(r, dst + off);
#pragma unroll
            for (int q = 0; q < 8; ++q) r[q] = fmaf(s, acc[q], r[q]);
        } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) r[q] = s * acc[q];
        }
        finish_vec<8>(r, p, off);
        store_vec<8>(dst + off, r);
    }
}

// Edge-stream variant for rows of 16*VEC < D <= 32*VEC floats with scalar weights: a warp owns R consecutive
// destination rows (or one hub chunk) and walks their edges - which are contiguous in the CSR - as ONE stream.
// Row pointers of the batch come from one coalesced load, column ids / weights from one coalesced load per 32
// edges (the next tile is requested before the current one is consumed), and the feature gathers are issued EU
// edges at a time without regard to row boundaries: when the stream crosses into the next row the accumulator is
// written out (a store, nothing waits for it) and cleared.  A short row therefore costs one store and a
// warp-uniform branch instead of its own chain of three dependent memory latencies (row pointer -> ids ->
// features) and its own warp, and no gather slot is spent on padding a row up to EU edges.  Rows that the hub
// schedule cuts into chunks are stepped over (their edges are neither loaded nor gathered).  Sums are formed in
// edge order, so results are run-to-run identical.
// Measured and not kept: a warp walking several batches in a row with the next batch's row pointers and first index tile
// requested ahead (7.0 / 7.3 / 7.8 / 8.6 ms for 1 / 2 / 4 / 8 batches against 5.64 ms on a 7.27 M-row, 65 M-edge shard: more
// state, spills at 80 registers, and fewer, longer-lived warps hide less latency); 16 edges per gather step (128 registers,
// 16 resident warps: 10.4 ms).
template <int VEC, int EU, int R, bool HUB, bool IDX32>
__global__ void __launch_bounds__(128, (VEC * EU <= 32) ? 6 : 4) spmm_stream_kernel(const __grid_constant__ SpmmParams p) {
    static_assert(R >= 1 && R <= 31 && EU >= 1 && EU <= 16 && 32 % EU == 0, "batch / unroll out of range");
    constexpr unsigned FULL = 0xffffffffu;
    constexpr unsigned GM = (1u << EU) - 1u;
    const int lane = threadIdx.x & 31;
    const int64_t gid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;

    // rp: first edge of row `lane` of the batch, relative to the batch's first edge (positions inside a batch fit 32
    // bits: the launcher sends graphs of 2^31 or more edges to the warp-per-row kernel)
    int64_t r0, E0;
    int nr, rp;
    bool raw;
    if (gid < p.chunk_tasks) {  // one chunk of a hub row: a one-row batch whose sum goes to scratch
        raw = true;
        nr = 1;
        r0 = __ldg(p.chunk_row + gid);
        E0 = __ldg(p.chunk_begin + gid);
        const int64_t rend = load_ptr(p.indptr, p.is64, r0 + 1);
        rp = lane == 0 ? 0 : static_cast<int>(min(static_cast<int64_t>(p.chunk_edges), rend - E0));
    } else {
        raw = false;
        r0 = (gid - p.chunk_tasks) * R;
        if (r0 >= p.row_tasks) return;
        nr = static_cast<int>(min(static_cast<int64_t>(R), p.n_rows - r0));
        const int64_t myptr = load_ptr(p.indptr, p.is64, r0 + min(lane, nr));
        E0 = __shfl_sync(FULL, myptr, 0);
        rp = static_cast<int>(myptr - E0);
    }
    const int len = __shfl_sync(FULL, rp, nr);  // edges of the batch
    const int rp_next = __shfl_down_sync(FULL, rp, 1);  // end of row `lane` (lanes < nr)
    const bool myhub = HUB && !raw && lane < nr && (rp_next - rp) > p.chunk_edges;
    const unsigned hub_rows = HUB ? __ballot_sync(FULL, myhub) : 0u;
    const int *idx = p.indices + E0;

    const int off = lane * VEC;
    const bool valid = off < p.D;
    float acc[VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] = 0.0f;

    auto load_tile = [&](int t, int &col, float &w) {
        col = 0;
        w = 0.0f;
        const int te = t + lane;
        if (te < len) {
            const int rawidx = ld_stream(idx + te);
            col = p.mask ? (rawidx & p.mask) : rawidx;
            if (p.wmode == YITU_W_NONE) {
                w = 1.0f;
            } else if (p.wmode == YITU_W_NODE) {
                w = __ldg(p.norm_src + col);  // the destination's factor is applied once per row, at the end
            } else {
                const int64_t ee = E0 + te;
                const int64_t vi = p.perm ? static_cast<int64_t>(ld_stream(p.perm + ee)) : ee;
                w = ld_stream(p.values + vi);
            }
        }
    };

    int cur = 0;  // row of the batch that the stream is in
    int cur_begin = 0, cur_end = __shfl_sync(FULL, rp, 1);
    // writes out every row that ends at or before position t (several when empty rows follow); warp-uniform
    auto flush = [&](int t) {
        while (cur < nr && cur_end <= t) {
            const int64_t row = r0 + cur;
            if (raw) {
                if (valid) {
                    if (p.wmode == YITU_W_NODE) {  // the reduction over chunks expects fully weighted partial sums
                        const float nd = __ldg(p.norm_dst + row);
#pragma unroll
                        for (int q = 0; q < VEC; ++q) acc[q] *= nd;
                    }
                    store_vec<VEC>(p.scratch + gid * p.D + off, acc);
                }
            } else if (!((hub_rows >> cur) & 1u)) {
                const bool had = cur_end > cur_begin;
                if (valid && (had || !p.accumulate || p.bias || p.act)) {
                    float s = p.alpha * (p.row_scale ? __ldg(p.row_scale + row) : 1.0f);
                    if (p.wmode == YITU_W_NODE) s *= __ldg(p.norm_dst + row);
                    float *dst = p.out + row * p.os + off;
                    float r[VEC];
                    if (p.accumulate) {
                        load_vec<VEC>(r, dst);
#pragma unroll
                        for (int q = 0; q < VEC; ++q) r[q] = fmaf(s, acc[q], r[q]);
                    } else {
#pragma unroll
                        for (int q = 0; q < VEC; ++q) r[q] = s * acc[q];
                    }
                    finish_vec<VEC>(r, p, off);
                    store_vec<VEC>(dst, r);
                }
            }
#pragma unroll
            for (int q = 0; q < VEC; ++q) acc[q] = 0.0f;
            ++cur;
            cur_begin = cur_end;
            cur_end = __shfl_sync(FULL, rp, min(cur + 1, 31));
        }
    };

    auto gather = [&](float (&v)[VEC], int c) {
        if (valid) {
            if constexpr (IDX32)
                load_vec<VEC>(v, p.x + (static_cast<uint32_t>(c) * static_cast<uint32_t>(p.xs) + static_cast<uint32_t>(off)));
            else
                load_vec<VEC>(v, p.x + static_cast<int64_t>(c) * p.xs + off);
        } else {
#pragma unroll
            for (int q = 0; q < VEC; ++q) v[q] = 0.0f;
        }
    };

    int t0 = 0;
    int my_col;
    float my_w;
    load_tile(t0, my_col, my_w);
    while (t0 < len) {
        const int n = min(32, len - t0);
        const int t_next = t0 + 32;
        int nx_col = 0;
        float nx_w = 0.0f;
        if (t_next < len) load_tile(t_next, nx_col, nx_w);
        // bm: positions of this tile where a row of the batch begins; hm: positions inside hub rows
        unsigned bm = 0u, hm = 0u;
        if (lane >= 1 && lane < nr) {
            const int d = rp - t0;
            if (d >= 0 && d < n) bm = 1u << d;
        }
        bm = __reduce_or_sync(FULL, bm);
        if constexpr (HUB) {
            if (myhub) {
                const int lo = max(rp - t0, 0), hi = min(rp_next - t0, n);
                if (hi > lo) hm = (hi - lo >= 32 ? FULL : ((1u << (hi - lo)) - 1u)) << lo;
            }
            hm = __reduce_or_sync(FULL, hm);
        }
        const unsigned vm = (n == 32 ? FULL : ((1u << n) - 1u)) & ~hm;
        if (HUB && vm == 0u) {
            // every edge of the tile belongs to hub rows: continue behind the hub row that holds the tile's last edge
            const int last = t0 + n - 1;
            const unsigned who = __ballot_sync(FULL, myhub && rp <= last && rp_next > last);
            t0 = __shfl_sync(FULL, rp_next, __ffs(who) - 1);
            if (t0 == t_next) {
                my_col = nx_col;
                my_w = nx_w;
            } else if (t0 < len) {
                load_tile(t0, my_col, my_w);
            }
            continue;
        }
        for (int j = 0; j < n; j += EU) {
            const unsigned gv = (vm >> j) & GM, gb = (bm >> j) & GM;
            if (HUB && gv == 0u && gb == 0u) continue;  // a group wholly inside a hub row
            int c[EU];
            float w[EU];
#pragma unroll
            for (int u = 0; u < EU; ++u) {
                c[u] = __shfl_sync(FULL, my_col, j + u);
                w[u] = __shfl_sync(FULL, my_w, j + u);
            }
            float v[EU][VEC];
            if (gv == GM && gb == 0u) {  // EU edges of one row: the common case
#pragma unroll
                for (int u = 0; u < EU; ++u) gather(v[u], c[u]);
#pragma unroll
                for (int u = 0; u < EU; ++u)
#pragma unroll
                    for (int q = 0; q < VEC; ++q) acc[q] = fmaf(w[u], v[u][q], acc[q]);
            } else {  // a row ends inside the group, or some positions carry no edge: same loads, uniform predicates
#pragma unroll
                for (int u = 0; u < EU; ++u)
                    if ((gv >> u) & 1u) gather(v[u], c[u]);
#pragma unroll
                for (int u = 0; u < EU; ++u) {
                    if ((gb >> u) & 1u) flush(t0 + j + u);
                    if ((gv >> u) & 1u) {
#pragma unroll
                        for (int q = 0; q < VEC; ++q) acc[q] = fmaf(w[u], v[u][q], acc[q]);
                    }
                }
            }
        }
        t0 = t_next;
        my_col = nx_col;
        my_w = nx_w;
    }
    flush(INT32_MAX);
}

// Adds the chunk partials of each hub row in chunk order and applies the epilogue.
__global__ void __launch_bounds__(128) hub_reduce_kernel(const __grid_constant__ SpmmParams p) {
    const int64_t chunk = blockIdx.x;
    const int64_t row = __ldg(p.chunk_row + chunk);
    const int64_t rb = load_ptr(p.indptr, p.is64, row);
    if (__ldg(p.chunk_begin + chunk) != rb) return;  // only a row's first chunk reduces
    const int64_t re = load_ptr(p.indptr, p.is64, row + 1);
    const int64_t nch = (re - rb + p.chunk_edges - 1) / p.chunk_edges;
    const float s = p.alpha * (p.row_scale ? __ldg(p.row_scale + row) : 1.0f);
    for (int64_t d = threadIdx.x; d < p.D; d += blockDim.x) {
        float a = 0.0f;
        for (int64_t k = 0; k < nch; ++k) a += p.scratch[(chunk + k) * p.D + d];
        float *o = p.out + row * p.os + d;
        float r = p.accumulate ? fmaf(s, a, *o) : s * a;
        if (p.bias) r += __ldg(p.bias + d);
        *o = activate(r, p.act);
    }
}

// 128-thread CTAs: with 256 a CTA waits for its longest row and occupancy drops (measured 7.57 -> 6.98 ms on the
// D=256 R-MAT workload; 32/64/128/256 gave 6.86/7.21/6.98/7.57 ms and 128 was best over all workloads).
static int block_threads() { return 128; }

template <int LPR, int NV, int VEC, int EU, int EU_HEAD = 4>
static int launch(const SpmmParams &p, bool per_head, cudaStream_t st, bool reduce = true) {
    const int64_t groups = p.chunk_tasks + p.row_tasks;
    if (groups == 0) return YITU_OK;
    const int threads = block_threads();
    const int gpb = threads / LPR;
    const int64_t gx = (groups + gpb - 1) / gpb;
    const int64_t gy = (p.D + LPR * NV * VEC - 1) / (LPR * NV * VEC);
    YITU_REQUIRE(gx < (1ll << 31) && gy <= 65535, YITU_ERR_LIMIT, "spmm grid too large (%lld x %lld)",
                 (long long)gx, (long long)gy);
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    // element offsets into x fit 32 bits?
    const bool idx32 = VEC >= 4 && p.n_cols * p.xs < (1ll << 32);
    if (per_head) {  // per-head weights cost registers per gathered slice: those variants unroll 4 edges only
        if (idx32) spmm_kernel<LPR, NV, VEC, EU_HEAD, true, true><<<grid, threads, 0, st>>>(p);
        else spmm_kernel<LPR, NV, VEC, EU_HEAD, true, false><<<grid, threads, 0, st>>>(p);
    } else {
        if (idx32) spmm_kernel<LPR, NV, VEC, EU, false, true><<<grid, threads, 0, st>>>(p);
        else spmm_kernel<LPR, NV, VEC, EU, false, false><<<grid, threads, 0, st>>>(p);
    }
    YITU_LAUNCH_CHECK();
    if (reduce && p.n_chunks > 0) {
        hub_reduce_kernel<<<static_cast<unsigned>(p.n_chunks), 128, 0, st>>>(p);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

template <int VEC, int EU, int R>
static int launch_stream(const SpmmParams &p, cudaStream_t st) {  // always followed by the hub reduction, if any
    const int64_t groups = p.chunk_tasks + (p.row_tasks + R - 1) / R;
    if (groups == 0) return YITU_OK;
    const int threads = block_threads();
    const int64_t gx = (groups + threads / 32 - 1) / (threads / 32);
    YITU_REQUIRE(gx < (1ll << 31), YITU_ERR_LIMIT, "spmm grid too large (%lld)", (long long)gx);
    const unsigned grid = static_cast<unsigned>(gx);
    const bool idx32 = p.n_cols * p.xs < (1ll << 32);
    const bool hub = p.n_chunks > 0;
    if (hub) {
        if (idx32) spmm_stream_kernel<VEC, EU, R, true, true><<<grid, threads, 0, st>>>(p);
        else spmm_stream_kernel<VEC, EU, R, true, false><<<grid, threads, 0, st>>>(p);
    } else {
        if (idx32) spmm_stream_kernel<VEC, EU, R, false, true><<<grid, threads, 0, st>>>(p);
        else spmm_stream_kernel<VEC, EU, R, false, false><<<grid, threads, 0, st>>>(p);
    }
    YITU_LAUNCH_CHECK();
    if (hub) {
        hub_reduce_kernel<<<static_cast<unsigned>(p.n_chunks), 128, 0, st>>>(p);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

// Development switches read from the environment at every call (measurement of one kernel form against another):
// YITU_SPMM_STREAM=0 keeps the warp-per-row kernels for every graph, =2 takes the edge-stream kernel for every graph
// whose shape it covers (default 1: by average row length, see yitu_spmm_csr_f32); YITU_SPMM_STREAM_ROWS=8|16|31 and
// YITU_SPMM_STREAM_EU pick an instantiation of the edge-stream kernel other than the default.
static int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

template <int VEC, int EU_A, int EU_B>
static int dispatch_stream(const SpmmParams &p, cudaStream_t st, int rows_dflt, int eu_dflt) {
    const int rows = env_int("YITU_SPMM_STREAM_ROWS", rows_dflt);
    const int eu = env_int("YITU_SPMM_STREAM_EU", eu_dflt);
    if (eu == EU_B) {
        if (rows == 8) return launch_stream<VEC, EU_B, 8>(p, st);
        if (rows == 31) return launch_stream<VEC, EU_B, 31>(p, st);
        return launch_stream<VEC, EU_B, 16>(p, st);
    }
    if (rows == 8) return launch_stream<VEC, EU_A, 8>(p, st);
    if (rows == 31) return launch_stream<VEC, EU_A, 31>(p, st);
    return launch_stream<VEC, EU_A, 16>(p, st);
}

template <int LPE, int EU>
static int launch_wide(const SpmmParams &p, cudaStream_t st) {
    const int64_t groups = p.chunk_tasks + p.row_tasks;
    if (groups == 0) return YITU_OK;
    const int threads = block_threads();
    const int64_t gx = (groups + threads / 32 - 1) / (threads / 32);
    YITU_REQUIRE(gx < (1ll << 31), YITU_ERR_LIMIT, "spmm grid too large (%lld)", (long long)gx);
    if (p.n_cols * p.xs < (1ll << 32)) spmm_wide_kernel<LPE, EU, true><<<static_cast<unsigned>(gx), threads, 0, st>>>(p);
    else spmm_wide_kernel<LPE, EU, false><<<static_cast<unsigned>(gx), threads, 0, st>>>(p);
    YITU_LAUNCH_CHECK();
    if (p.n_chunks > 0) {
        hub_reduce_kernel<<<static_cast<unsigned>(p.n_chunks), 128, 0, st>>>(p);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

}  // namespace yitu

using namespace yitu;

extern "C" int yitu_spmm_csr_f32(const yitu_spmm_args_t *a, yitu_stream_t stream) {
    YITU_REQUIRE(a != nullptr, YITU_ERR_INVALID_ARG, "args is NULL");
    if (int rc = validate_csr(&a->graph)) return rc;
    const yitu_csr_t &g = a->graph;
    YITU_REQUIRE(a->n_heads >= 1 && a->n_feats >= 1, YITU_ERR_INVALID_ARG, "n_heads=%lld n_feats=%lld",
                 (long long)a->n_heads, (long long)a->n_feats);
    const int64_t D = a->n_heads * a->n_feats;
    YITU_REQUIRE(a->x_shared_heads == 0 || a->weight_mode == YITU_W_EDGE_HEAD, YITU_ERR_INVALID_ARG,
                 "x_shared_heads needs per-head edge values (YITU_W_EDGE_HEAD)");
    const int64_t x_width = a->x_shared_heads ? a->n_feats : D;
    YITU_REQUIRE(a->x_stride >= x_width && a->out_stride >= D, YITU_ERR_INVALID_ARG,
                 "row strides (%lld, %lld) smaller than the rows (%lld, %lld)", (long long)a->x_stride,
                 (long long)a->out_stride, (long long)x_width, (long long)D);
    YITU_REQUIRE(a->activation >= YITU_ACT_NONE && a->activation <= YITU_ACT_ELU, YITU_ERR_INVALID_ARG,
                 "unknown activation %d", a->activation);
    YITU_REQUIRE(g.n_rows == 0 || a->out != nullptr, YITU_ERR_INVALID_ARG, "out is NULL");
    YITU_REQUIRE(g.nnz == 0 || a->x != nullptr, YITU_ERR_INVALID_ARG, "x is NULL");
    YITU_REQUIRE(a->weight_mode >= YITU_W_NONE && a->weight_mode <= YITU_W_EDGE_HEAD, YITU_ERR_INVALID_ARG,
                 "unknown weight_mode %d", a->weight_mode);
    if (a->weight_mode == YITU_W_NODE)
        YITU_REQUIRE(a->norm_dst && a->norm_src, YITU_ERR_INVALID_ARG, "W_NODE needs norm_dst and norm_src");
    if (a->weight_mode == YITU_W_EDGE || a->weight_mode == YITU_W_EDGE_HEAD)
        YITU_REQUIRE(g.nnz == 0 || a->edge_values, YITU_ERR_INVALID_ARG, "edge_values is NULL");
    const bool per_head = a->weight_mode == YITU_W_EDGE_HEAD;
    if (per_head)
        YITU_REQUIRE(g.nnz < (1ll << 31), YITU_ERR_LIMIT, "per-head edge values need nnz < 2^31");

    SpmmParams p{};
    p.n_rows = g.n_rows; p.n_cols = g.n_cols; p.D = D; p.H = a->n_heads; p.F = a->n_feats;
    p.indptr = g.indptr; p.indices = g.indices; p.is64 = g.indptr_is64; p.mask = g.index_mask;
    p.wmode = a->weight_mode; p.accumulate = a->accumulate;
    p.values = a->edge_values; p.perm = a->edge_perm;
    p.norm_dst = a->norm_dst; p.norm_src = a->norm_src; p.row_scale = a->row_scale; p.alpha = a->alpha;
    p.x = a->x; p.xs = a->x_stride; p.out = a->out; p.os = a->out_stride;
    p.bias = a->bias; p.act = a->activation; p.xshared = a->x_shared_heads ? 1 : 0;
    p.row_tasks = g.n_rows;
    if (a->plan && a->plan->n_chunks > 0) {
        YITU_REQUIRE(a->plan->chunk_edges >= 32, YITU_ERR_INVALID_ARG, "plan.chunk_edges must be >= 32");
        YITU_REQUIRE(a->plan->chunk_row && a->plan->chunk_begin, YITU_ERR_INVALID_ARG, "plan tables are NULL");
        YITU_REQUIRE(a->scratch != nullptr && a->scratch_bytes >= a->plan->n_chunks * D * 4, YITU_ERR_WORKSPACE,
                     "scratch needs %lld bytes, got %lld", (long long)(a->plan->n_chunks * D * 4),
                     (long long)a->scratch_bytes);
        p.n_chunks = a->plan->n_chunks; p.chunk_tasks = p.n_chunks; p.chunk_edges = a->plan->chunk_edges;
        p.chunk_row = a->plan->chunk_row; p.chunk_begin = a->plan->chunk_begin; p.scratch = a->scratch;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

    const bool vec_ok = (D % 4 == 0) && (a->x_stride % 4 == 0) && (a->out_stride % 4 == 0) && aligned16(a->x) &&
                        aligned16(a->out) && (p.scratch == nullptr || aligned16(p.scratch)) &&
                        (!per_head || a->n_feats % 4 == 0);
    if (!vec_ok) return launch<32, 4, 1, 4>(p, per_head, st);
    // lanes per row / 128-bit slices per lane / edges gathered per step, from a sweep on B200: narrower groups
    // than the row lose coalescing; deeper unrolling pays while it fits the register budget
    // rows of more than 128 floats: 256-bit loads (one 1 KiB request per warp and edge) when everything is 32-byte
    // aligned; measured 6.20 ms against 6.44 ms with 128-bit loads on the D=256 R-MAT workload.  Narrower rows would
    // need half-warp groups, which lose more than the wider loads gain.
    const auto aligned32 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0; };
    // YITU_SPMM_STREAM (development switch): 0 warp-per-row kernel for everything; 2 edge-stream kernel for everything it
    // covers, hub chunks included; 3 one of the two by average row length (stream below 24 edges per row);
    // 1 (default) both: the chunks of the hub rows go to the warp-per-row kernel - long uniform tasks, where its 32
    // resident warps at 64 registers win - and all other rows to the edge-stream kernel, in two launches on the stream;
    // for graphs below 64 edges per row (24 for rows of more than 128 floats), the warp-per-row kernel alone above.
    // Measured on B200, 128 features (ms: warp per row / both / stream alone): R-MAT 16.8 M rows x 31 edges 34.70 /
    // 32.60 / 35.00; its 8-way shards of 65 M edges each: 7.27 M rows 6.49 / 5.51 / 5.64, 3.07 M rows 4.89 / 4.61 / 4.76,
    // 1.20 M rows 4.17 / 4.23 / 4.41, 82 k rows (795 per row) 3.43 / 3.68 / 4.03.  256 features, 2.1 M rows x 30: 6.08 /
    // 6.17 / 6.18.  Uniform graph, 16 edges per row, no hubs: 11.83 / - / 10.74.
    const int stream_mode = env_int("YITU_SPMM_STREAM", 1);
    const bool stream_shape = !per_head && g.nnz < (1ll << 31);
    const bool stream_ok = stream_shape && (stream_mode == 2 || (stream_mode == 3 && g.nnz < 24 * g.n_rows));
    const bool split = stream_shape && stream_mode == 1 && g.nnz < (D > 128 ? 24 : 64) * g.n_rows;
    const bool wide256 = D > 128 && D <= 256 && D % 8 == 0 && a->x_stride % 8 == 0 && a->out_stride % 8 == 0 &&
                         aligned32(a->x) && aligned32(a->out) && (p.scratch == nullptr || aligned32(p.scratch));
    if (split && (wide256 || (D > 64 && D <= 128))) {
        if (p.n_chunks > 0) {
            SpmmParams c = p;
            c.row_tasks = 0;  // the chunks only; the reduction follows the second launch
            if (int rc = wide256 ? launch<32, 1, 8, 4>(c, false, st, false) : launch<32, 1, 4, 16>(c, false, st, false)) return rc;
        }
        SpmmParams r = p;
        r.chunk_tasks = 0;  // the rows that are not cut into chunks (those are stepped over), then the reduction
        return wide256 ? dispatch_stream<8, 4, 8>(r, st, 16, 4) : dispatch_stream<4, 8, 16>(r, st, 16, 8);
    }
    if (stream_ok && wide256) return dispatch_stream<8, 4, 8>(p, st, 16, 4);
    if (stream_ok && D > 64 && D <= 128) return dispatch_stream<4, 8, 16>(p, st, 16, 8);
    if (D > 128 && D <= 512 && D % 8 == 0 && a->x_stride % 8 == 0 && a->out_stride % 8 == 0 && aligned32(a->x) &&
        aligned32(a->out) && (p.scratch == nullptr || aligned32(p.scratch)) && (!per_head || a->n_feats % 8 == 0)) {
        if (D <= 256) return launch<32, 1, 8, 4>(p, per_head, st);
        return launch<32, 2, 8, 4>(p, per_head, st);
    }
    // rows of 33..64 floats with scalar weights: a full warp per row, four edges per 256-bit load instruction
    // (measured 0.350 ms against 0.392 ms for half-warp rows on the D=64 hetero workload; for 65..128 floats the same
    // scheme lost, 37.5 ms against 34.6 ms)
    if (!per_head && D > 32 && D <= 64 && D % 8 == 0 && a->x_stride % 8 == 0 && a->out_stride % 8 == 0 && aligned32(a->x) &&
        aligned32(a->out) && (p.scratch == nullptr || aligned32(p.scratch)))
        return launch_wide<8, 1>(p, st);
    if (D <= 16) return launch<4, 1, 4, 4>(p, per_head, st);
    if (D <= 32) return launch<8, 1, 4, 4>(p, per_head, st);
    if (D <= 64) return launch<16, 1, 4, 4>(p, per_head, st);
    if (D <= 128) return launch<32, 1, 4, 16>(p, per_head, st);
    if (D <= 256) return launch<32, 2, 4, 8>(p, per_head, st);
    return launch<32, 4, 4, 4>(p, per_head, st);
}
