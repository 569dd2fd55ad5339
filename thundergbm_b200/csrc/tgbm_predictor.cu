// Batch inference: Predictor::predict_raw (src/thundergbm/predictor.cu:32-189), the objectives'
// predict_transform and the metric the predict CLI logs.
#include <algorithm>
#include <cmath>

#include "tgbm_booster.h"
#include "tgbm_kernels.cuh"
#include "tgbm_rank.cuh"

namespace tgbm {

// 16-byte traversal record (the 48-byte model record carries training-only fields)
struct PNode {
    float v;     // split value, or leaf weight
    int fid;     // feature id; bit 31 = leaf, bit 30 = default right
    int lch, rch;
};

constexpr int PRED_ROWS = 128;

// Rows of a tile are densified in shared memory (INFINITY = missing), one thread walks every tree of
// every class for its row.  The reference takes this path when F*128*4 <= 48 KB and accumulates in
// double from base_score, adding the result to a zeroed float (predictor.cu:88-134).
__global__ void __launch_bounds__(PRED_ROWS)
k_predict_dense(const int *__restrict__ row_ptr, const int *__restrict__ col, const float *__restrict__ val, int n_rows, int F,
                const PNode *__restrict__ model, int n_rounds, int K, int n_nodes, float lr, float base_score,
                float *__restrict__ out) {
    extern __shared__ float dense[];  // [F][PRED_ROWS]
    const int i = blockIdx.x * PRED_ROWS + threadIdx.x;
    for (int f = 0; f < F; ++f) dense[f * PRED_ROWS + threadIdx.x] = INFINITY;
    if (i < n_rows)
        for (int j = row_ptr[i]; j < row_ptr[i + 1]; ++j) {
            const int c = col[j];
            if (c < F) dense[c * PRED_ROWS + threadIdx.x] = val[j];
        }
    if (i >= n_rows) return;
    for (int t = 0; t < K; ++t) {
        double sum = base_score;
        for (int r = 0; r < n_rounds; ++r) {
            const PNode *nd = model + ((size_t)r * K + t) * n_nodes;
            PNode cur = nd[0];
            while (!(cur.fid & 0x80000000)) {
                const int f = cur.fid & 0x3fffffff;
                const float fv = f < F ? dense[f * PRED_ROWS + threadIdx.x] : INFINITY;
                int nx;
                if (fv < INFINITY) nx = fv < cur.v ? cur.lch : cur.rch;
                else nx = (cur.fid & 0x40000000) ? cur.rch : cur.lch;
                cur = nd[nx];
            }
            sum += (double)__fmul_rn(lr, cur.v);
        }
        out[(size_t)t * n_rows + i] = (float)(0.0 + sum);
    }
}

// CSR path with a binary search per visited node; float accumulator, `sum += lr * w` is one fused
// multiply-add in the reference's compiled code (predictor.cu:137-187)
__global__ void k_predict_csr(const int *__restrict__ row_ptr, const int *__restrict__ col, const float *__restrict__ val, int n_rows,
                              const PNode *__restrict__ model, int n_rounds, int K, int n_nodes, float lr, float base_score,
                              float *__restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows) return;
    const int *ci = col + row_ptr[i];
    const float *vi = val + row_ptr[i];
    const int len = row_ptr[i + 1] - row_ptr[i];
    for (int t = 0; t < K; ++t) {
        float sum = base_score;
        for (int r = 0; r < n_rounds; ++r) {
            const PNode *nd = model + ((size_t)r * K + t) * n_nodes;
            PNode cur = nd[0];
            while (!(cur.fid & 0x80000000)) {
                const int f = cur.fid & 0x3fffffff;
                int lo = 0, hi = len;
                bool found = false;
                float fv = 0.f;
                while (lo != hi) {
                    const int mid = lo + (hi - lo) / 2;
                    const int c = ci[mid];
                    if (c == f) { found = true; fv = vi[mid]; break; }
                    if (c > f) hi = mid; else lo = mid + 1;
                }
                int nx;
                if (found) nx = fv < cur.v ? cur.lch : cur.rch;
                else nx = (cur.fid & 0x40000000) ? cur.rch : cur.lch;
                cur = nd[nx];
            }
            sum = __fmaf_rn(lr, cur.v, sum);
        }
        out[(size_t)t * n_rows + i] = sum;
    }
}

// The CSR path's arithmetic (float accumulator, fused multiply-add per tree) with the lookups of the dense path: the
// rows of a tile are spread out in shared memory first, so that a visited node costs one shared-memory read instead
// of a binary search through the row in global memory.  Used when the reference would take its CSR path
// (F * 128 * 4 > 48 KB) and a tile still fits the 227 KB of a B200 SM.  A slot holding PRED_ABSENT was never stored.
constexpr unsigned PRED_ABSENT = 0x7fc00b20u;  // a quiet NaN with a payload no computation produces
__global__ void __launch_bounds__(PRED_ROWS)
k_predict_csr_staged(const int *__restrict__ row_ptr, const int *__restrict__ col, const float *__restrict__ val, int n_rows, int F,
                     const PNode *__restrict__ model, int n_rounds, int K, int n_nodes, float lr, float base_score,
                     float *__restrict__ out) {
    extern __shared__ float dense[];  // [F][PRED_ROWS]
    const int i = blockIdx.x * PRED_ROWS + threadIdx.x;
    for (int f = 0; f < F; ++f) dense[f * PRED_ROWS + threadIdx.x] = __uint_as_float(PRED_ABSENT);
    if (i >= n_rows) return;
    for (int j = row_ptr[i]; j < row_ptr[i + 1]; ++j) {
        const int c = col[j];
        if (c >= 0 && c < F) dense[c * PRED_ROWS + threadIdx.x] = val[j];
    }
    for (int t = 0; t < K; ++t) {
        float sum = base_score;
        for (int r = 0; r < n_rounds; ++r) {
            const PNode *nd = model + ((size_t)r * K + t) * n_nodes;
            PNode cur = nd[0];
            while (!(cur.fid & 0x80000000)) {
                const int f = cur.fid & 0x3fffffff;
                const float fv = f < F ? dense[f * PRED_ROWS + threadIdx.x] : __uint_as_float(PRED_ABSENT);
                int nx;
                if (__float_as_uint(fv) != PRED_ABSENT) nx = fv < cur.v ? cur.lch : cur.rch;
                else nx = (cur.fid & 0x40000000) ? cur.rch : cur.lch;
                cur = nd[nx];
            }
            sum = __fmaf_rn(lr, cur.v, sum);
        }
        out[(size_t)t * n_rows + i] = sum;
    }
}


// ---- tiled traversal ---------------------------------------------------------------------------------------------
// The same two arithmetics (dense path: double accumulator, missing = +inf; CSR path: float accumulator with one fused
// multiply-add per tree, missing = a slot never stored) with everything a step touches in shared memory:
//   * the trees of a chunk as 8-byte records in heap order (the node table IS a heap: children of i are 2i+1, 2i+2,
//     checked on the host), so a step is one 8-byte read of the node and one 4-byte read of the row's feature;
//   * the rows of a tile spread out as [feature][row] (bank = row: no conflicts whatever features the lanes ask for);
//   * 512 threads per CTA, RPT rows per thread walk a tree level by level side by side -- a walk is a chain of
//     dependent shared-memory reads, many independent chains keep the pipeline busy.
// Trees are visited in ascending round order for every row, so the sums are those of the one-thread-per-row kernels
// bit for bit.  CTAs are persistent and loop over the row tiles.
struct HNode { float v; int fid; };  // split value or leaf weight; feature id, bit 31 = leaf, bit 30 = default right
constexpr int PT_THREADS = 512;

template <bool DENSE_PATH, int RPT>
__global__ void __launch_bounds__(PT_THREADS)
k_predict_tiles(const int *__restrict__ row_ptr, const int *__restrict__ col, const float *__restrict__ val, int n_rows, int F,
                const HNode *__restrict__ model, int n_rounds, int K, int n_nodes, int depth, int chunk_trees, float lr,
                float base_score, float *__restrict__ out, double *__restrict__ partial) {
    // Loop order: class, chunk of trees (staged once per CTA), the CTA's row tiles.  With more than one chunk the running
    // sums of a row wait in `partial` (double [K][n_rows]; the CSR path keeps its float there) between the chunks, so that
    // every row still adds its trees in ascending round order.
    extern __shared__ __align__(16) unsigned char pt_sm[];
    constexpr int ROWS = PT_THREADS * RPT;
    float *dense = reinterpret_cast<float *>(pt_sm);                                   // [F][ROWS]
    HNode *trees = reinterpret_cast<HNode *>(pt_sm + sizeof(float) * (size_t)F * ROWS);  // [chunk_trees][n_nodes]
    const float absent = DENSE_PATH ? INFINITY : __uint_as_float(PRED_ABSENT);
    const int n_tiles = (n_rows + ROWS - 1) / ROWS;
    for (int t = 0; t < K; ++t) {
        for (int r0 = 0; r0 < n_rounds; r0 += chunk_trees) {
            const int nc = min(chunk_trees, n_rounds - r0);
            const bool first = r0 == 0, last = r0 + nc >= n_rounds;
            __syncthreads();  // the previous chunk's walks are over
            for (int i = threadIdx.x; i < nc * n_nodes; i += PT_THREADS)
                trees[i] = model[((size_t)(r0 + i / n_nodes) * K + t) * n_nodes + i % n_nodes];
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                __syncthreads();  // the previous tile's walks are over (and the trees are in place)
                const int row0 = tile * ROWS;
                for (int i = threadIdx.x; i < F * ROWS; i += PT_THREADS) dense[i] = absent;
                __syncthreads();
                // A thread spreads out its own rows: the slots it writes are its own column of `dense` (bank = row: no
                // conflicts), neighbouring threads read neighbouring rows (whole cache lines get used), and the loads
                // are issued in batches of eight so that the few warps of the CTA cover the memory latency.
                constexpr int BATCH = 8;
#pragma unroll
                for (int j = 0; j < RPT; ++j) {
                    const int q = j * PT_THREADS + threadIdx.x, i = row0 + q;
                    if (i >= n_rows) continue;
                    const int ea = row_ptr[i], ez = row_ptr[i + 1];
                    for (int eb = ea; eb < ez; eb += BATCH) {
                        int cc[BATCH];
                        float vv[BATCH];
#pragma unroll
                        for (int u = 0; u < BATCH; ++u) {
                            cc[u] = eb + u < ez ? col[eb + u] : -1;
                            vv[u] = eb + u < ez ? val[eb + u] : 0.f;
                        }
#pragma unroll
                        for (int u = 0; u < BATCH; ++u)
                            if (cc[u] >= 0 && cc[u] < F) dense[cc[u] * ROWS + q] = vv[u];
                    }
                }
                // the next tile's values on their way into L2 while this one is walked
                if (tile + (int)gridDim.x < n_tiles) {
                    const int nr0 = min(row0 + (int)gridDim.x * ROWS, n_rows), nr1 = min(nr0 + ROWS, n_rows);
                    const int ne0 = row_ptr[nr0], ne1 = row_ptr[nr1];
                    for (int e = ne0 + threadIdx.x * 32; e < ne1; e += PT_THREADS * 32) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(col + e));
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(val + e));
                    }
                }
                double dsum[RPT];
                float fsum[RPT];
#pragma unroll
                for (int j = 0; j < RPT; ++j) {
                    const int i = row0 + j * PT_THREADS + threadIdx.x;
                    dsum[j] = base_score; fsum[j] = base_score;
                    if (i < n_rows && !first) {
                        const double p = partial[(size_t)t * n_rows + i];
                        dsum[j] = p; fsum[j] = (float)p;  // a float survives the round trip through a double unchanged
                    }
                }
                __syncthreads();
                for (int c = 0; c < nc; ++c) {
                    const HNode *nd = trees + (size_t)c * n_nodes;
                    int cur[RPT];
#pragma unroll
                    for (int j = 0; j < RPT; ++j) cur[j] = 0;
                    for (int lvl = 0; lvl < depth; ++lvl) {
                        HNode h[RPT];
#pragma unroll
                        for (int j = 0; j < RPT; ++j) h[j] = nd[cur[j]];
                        float fv[RPT];
#pragma unroll
                        for (int j = 0; j < RPT; ++j) fv[j] = dense[min(h[j].fid & 0x3fffffff, F - 1) * ROWS + j * PT_THREADS + threadIdx.x];
#pragma unroll
                        for (int j = 0; j < RPT; ++j) {
                            const float v = (h[j].fid & 0x3fffffff) < F ? fv[j] : absent;
                            const bool present = DENSE_PATH ? (v < INFINITY) : (__float_as_uint(v) != PRED_ABSENT);
                            const bool right = present ? !(v < h[j].v) : (h[j].fid & 0x40000000) != 0;
                            cur[j] = h[j].fid >= 0 ? 2 * cur[j] + 1 + (right ? 1 : 0) : cur[j];
                        }
                    }
#pragma unroll
                    for (int j = 0; j < RPT; ++j) {
                        const float w = nd[cur[j]].v;
                        if (DENSE_PATH) dsum[j] += (double)__fmul_rn(lr, w);
                        else fsum[j] = __fmaf_rn(lr, w, fsum[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < RPT; ++j) {
                    const int i = row0 + j * PT_THREADS + threadIdx.x;
                    if (i >= n_rows) continue;
                    if (last) out[(size_t)t * n_rows + i] = DENSE_PATH ? (float)(0.0 + dsum[j]) : fsum[j];
                    else partial[(size_t)t * n_rows + i] = DENSE_PATH ? dsum[j] : (double)fsum[j];
                }
            }
        }
    }
}

template <bool DENSE_PATH>
static bool launch_predict_tiles(const int *rp, const int *col, const float *val, int N, int F, const HNode *model, int n_rounds, int K,
                                 int n_nodes, int depth, float lr, float base_score, float *out, int num_sms, cudaStream_t st,
                                 DevBuf<double> &partial, bool plan_only) {
    const size_t budget = 200 * 1024, tree_bytes = sizeof(HNode) * (size_t)n_nodes;
    // fewer rows per tile leave room for more trees per chunk, and every chunk is one more pass over the rows: take the
    // tile size that needs fewer passes (two rows per thread when it is a tie)
    auto passes = [&](int rpt) -> long {
        const size_t rows_bytes = sizeof(float) * (size_t)F * PT_THREADS * rpt;
        if (rows_bytes + std::min<size_t>(8, n_rounds) * tree_bytes > budget) return 1L << 40;
        const long chunk = (long)std::min<size_t>((size_t)n_rounds, (budget - rows_bytes) / tree_bytes);
        return (n_rounds + chunk - 1) / chunk;
    };
    const int order[2] = {passes(2) <= passes(1) ? 2 : 1, passes(2) <= passes(1) ? 1 : 2};
    for (int rpt : order) {
        const size_t rows_bytes = sizeof(float) * (size_t)F * PT_THREADS * rpt;
        if (rows_bytes + std::min<size_t>(8, n_rounds) * tree_bytes > budget) continue;  // at least 8 trees (or all) per chunk
        const int chunk = (int)std::min<size_t>((size_t)n_rounds, (budget - rows_bytes) / tree_bytes);
        const size_t smem = rows_bytes + chunk * tree_bytes;
        if (chunk < n_rounds && partial.n < (size_t)N * K) partial.alloc((size_t)N * K);  // running sums between the chunks
        if (plan_only) return true;
        const int tiles = (N + PT_THREADS * rpt - 1) / (PT_THREADS * rpt);
        const int grid = std::max(1, std::min(tiles, num_sms));
        auto go = [&](auto kern) {
            TGBM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kern<<<grid, PT_THREADS, smem, st>>>(rp, col, val, N, F, model, n_rounds, K, n_nodes, depth, chunk, lr, base_score, out, partial.p);
        };
        if (rpt == 2) go(k_predict_tiles<DENSE_PATH, 2>);
        else go(k_predict_tiles<DENSE_PATH, 1>);
        return true;
    }
    return false;
}


// ---- traversal on ranks ------------------------------------------------------------------------------------------
// A model compares feature values with a few hundred distinct thresholds per feature at most (it was trained on at
// most 255 bins).  With the thresholds of feature f sorted, s_0 < s_1 < ..., and r(v) = #{i : s_i <= v}, the test the
// reference makes at a node with threshold s_t,  v < s_t  (predictor.cu:89-91, :158-160), is exactly  r(v) <= t.  So
// every row is converted ONCE to one byte per feature (its rank, 255 = absent) and all trees are walked on bytes:
// a row of up to 32 features sits in 8 registers, the whole shared memory holds trees (8-byte records in heap order),
// and four rows per thread walk side by side.  Same comparisons, same order of the sums: the scores are those of the
// float kernels bit for bit.  Used when no feature has more than 254 thresholds and every tree is a heap.
struct RNode { int flags; float weight; };  // threshold rank (bits 0-7) | default right (8) | leaf (9) | feature << 16
constexpr int RK_ROWS = 512;     // rows of a block of k_rank_rows
constexpr int RK_THREADS = 256;

// CSR values -> ranks.  A block owns RK_ROWS consecutive rows = one contiguous piece of the CSR arrays; its warps read
// that piece 32 values at a time (coalesced) and find the row of every value in the block's row pointers: a 32-ary
// search for the warp's first value, then a walk over the few row boundaries inside the warp's 32 values.
// SMEM_THR: the thresholds sit in shared memory, 256 per feature padded with +inf at a stride of 257 floats (lanes on
// different features then hit different banks at every step), and the search is eight branch-free steps.
constexpr int RK_THR_STRIDE = 257;
template <bool DENSE_PATH, bool SMEM_THR>
__global__ void __launch_bounds__(RK_THREADS)
k_rank_rows(const int *__restrict__ row_ptr, const int *__restrict__ col, const float *__restrict__ val, int n_rows, int F, int Fpad,
            const int *__restrict__ thr_ptr, const float *__restrict__ thr, unsigned char *__restrict__ bins) {
    __shared__ int s_rp[RK_ROWS + 1];
    extern __shared__ float s_thr[];   // SMEM_THR: [F][RK_THR_STRIDE]
    if (SMEM_THR)   // once per block; the blocks are persistent
        for (int i = threadIdx.x; i < F * 256; i += RK_THREADS) {
            const int f = i >> 8, k = i & 255, a = thr_ptr[f];
            s_thr[f * RK_THR_STRIDE + k] = a + k < thr_ptr[f + 1] ? thr[a + k] : INFINITY;
        }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_tiles = (n_rows + RK_ROWS - 1) / RK_ROWS;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int row0 = tile * RK_ROWS;
    __syncthreads();   // the previous tile's row pointers have been read (and the thresholds are in place)
    for (int i = threadIdx.x; i <= RK_ROWS; i += RK_THREADS) s_rp[i] = row_ptr[min(row0 + i, n_rows)];
    __syncthreads();
    const int e0 = s_rp[0], e1 = s_rp[RK_ROWS];
    constexpr int UNROLL = 4;  // pieces of 32 values per warp and iteration: their loads are issued together
    for (int base0 = e0 + warp * 32 * UNROLL; base0 < e1; base0 += RK_THREADS * UNROLL) {
        int cc[UNROLL];
        float vv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int e = base0 + 32 * u + lane;
            cc[u] = e < e1 ? col[e] : -1;
            vv[u] = e < e1 ? val[e] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int base = base0 + 32 * u, e = base + lane;
            if (base >= e1) break;
            const int c = cc[u];
            const float v = vv[u];
            // row of the piece's first value: the last q with s_rp[q] <= base (RK_ROWS = 32 * 16)
            const int blk = __popc(__ballot_sync(0xffffffffu, s_rp[16 * lane] <= base)) - 1;
            const int q0 = 16 * blk + __popc(__ballot_sync(0xffffffffu, lane < 16 && s_rp[16 * blk + lane] <= base)) - 1;
            int q = q0;
            for (int k = 1; q0 + k <= RK_ROWS; ++k) {  // row boundaries inside the piece
                const int nb = s_rp[q0 + k];
                if (nb > base + 31) break;
                if (nb <= e) q = q0 + k;
            }
            if (c >= 0 && c < F) {
                int lo = thr_ptr[c];
                const int first = lo;
                int hi = thr_ptr[c + 1];
                const int n_thr = hi - first;
                if (SMEM_THR) {
                    const float *t = s_thr + c * RK_THR_STRIDE;
                    int pos = 0;
#pragma unroll
                    for (int step = 128; step >= 1; step >>= 1) pos += t[pos + step - 1] <= v ? step : 0;
                    lo = first + min(pos, n_thr);   // a stored +inf passes the padding too
                } else
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (thr[mid] <= v) lo = mid + 1; else hi = mid;
                }
                int r = lo - first;
                if (DENSE_PATH) { if (!(v < INFINITY)) r = 255; }  // the dense path marks absent features with +inf (predictor.cu:95)
                else if (v != v) r = n_thr;                         // no threshold is above a NaN: always right
                bins[(size_t)(row0 + q) * Fpad + c] = (unsigned char)r;
            }
        }
    }
    }
}

// Rows that store every feature, columns in order (a dense matrix handed over as CSR): one thread per row reads its F
// values with 16-byte loads, checks its row pointer and the column ids against 0 .. F-1 as it goes (any other row raises `not_dense` and
// the caller falls back to the kernel above) and ranks each value by an eight-step descent through the feature's
// thresholds laid out as an implicit search tree (level by level: the lanes of a warp, all on the same feature, touch
// consecutive words).  No row search, no address arithmetic per value: ncu counted 130 warp instructions per value in the
// kernel above.
constexpr int RD_THREADS = 256;
template <bool DENSE_PATH>
__global__ void __launch_bounds__(RD_THREADS)
k_rank_dense_rows(const int *__restrict__ row_ptr, const int *__restrict__ col, const float *__restrict__ val, int n_rows, int F, const float *__restrict__ tree_thr,
                  const int *__restrict__ thr_ptr, unsigned char *__restrict__ bins, int *__restrict__ not_dense) {
    extern __shared__ float s_tree[];   // [F][256]: 255 thresholds of the feature in level order, padded with +inf
    __shared__ int s_n[32];
    for (int i = threadIdx.x; i < F * 256; i += RD_THREADS) s_tree[i] = tree_thr[i];
    if (threadIdx.x < F) s_n[threadIdx.x] = thr_ptr[threadIdx.x + 1] - thr_ptr[threadIdx.x];
    __syncthreads();
    const int F4 = F / 4;   // F is a multiple of 4 here
    bool bad = false;
    for (int r = blockIdx.x * RD_THREADS + threadIdx.x; r < n_rows; r += gridDim.x * RD_THREADS) {
        const float4 *vp = reinterpret_cast<const float4 *>(val + (size_t)r * F);
        const int4 *cp = reinterpret_cast<const int4 *>(col + (size_t)r * F);
        bad |= row_ptr[r] != r * F;
        uint32_t out[8] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (q < F4) {
                const float4 v4 = vp[q];
                const int4 c4 = cp[q];
                bad |= c4.x != 4 * q || c4.y != 4 * q + 1 || c4.z != 4 * q + 2 || c4.w != 4 * q + 3;
                const float v[4] = {v4.x, v4.y, v4.z, v4.w};
                uint32_t word = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int f = 4 * q + k;
                    const float *t = s_tree + f * 256;
                    int pos = 0;
#pragma unroll
                    for (int step = 0; step < 8; ++step) pos = 2 * pos + (t[pos] <= v[k] ? 2 : 1);
                    int rank = min(pos - 255, s_n[f]);   // a stored +inf passes the padding too
                    if (DENSE_PATH) { if (!(v[k] < INFINITY)) rank = 255; }
                    else if (v[k] != v[k]) rank = s_n[f];
                    word |= (uint32_t)rank << (8 * k);
                }
                out[q] = word;
            }
        }
        uint4 *dst = reinterpret_cast<uint4 *>(bins + (size_t)r * 32);
        dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) *not_dense = 1;
}

constexpr int PR_THREADS = 512;
constexpr int PR_RPT = 4;
constexpr int PR_ROWS = PR_THREADS * PR_RPT;
// WORD_ROWS: rows of at most 32 features.  A row's eight 32-bit words are spread out in shared memory as [word][row]
// (bank = row: no conflicts whatever word a lane asks for) plus a ninth word of absent marks that nodes on features the
// data does not have point at; a step costs one read of the node's flags, one read of a word, a shift and a mask -- the
// kernel is bound by instruction issue, and picking a byte out of eight registers costs twice as many instructions.
// Otherwise the rank bytes are read from global memory (L1) at every step.
// Node flags: threshold rank (bits 0-7) | default right (8) | leaf (9) | bit offset of the byte in its word (10-14) |
// word index (WORD_ROWS) or feature id (16-31).
template <bool DENSE_PATH, bool WORD_ROWS>
__global__ void __launch_bounds__(PR_THREADS)
k_predict_ranks(const unsigned char *__restrict__ bins, int Fpad, int F, int n_rows, const RNode *__restrict__ model, int n_rounds, int K,
                int n_nodes, int depth, int chunk_trees, float lr, float base_score, float *__restrict__ out, double *__restrict__ partial) {
    extern __shared__ __align__(16) unsigned char rk_sm[];
    constexpr int RPT = PR_RPT, ROWS = PR_ROWS;
    uint32_t *words = reinterpret_cast<uint32_t *>(rk_sm);                          // [9][ROWS] (WORD_ROWS only)
    int *tflags = reinterpret_cast<int *>(rk_sm) + (WORD_ROWS ? 9 * ROWS : 0);      // [chunk_trees][n_nodes]
    float *tweight = reinterpret_cast<float *>(tflags) + (size_t)chunk_trees * n_nodes;
    const int n_tiles = (n_rows + ROWS - 1) / ROWS;
    if (WORD_ROWS)
        for (int i = threadIdx.x; i < ROWS; i += PR_THREADS) words[8 * ROWS + i] = 0xffffffffu;
    for (int t = 0; t < K; ++t) {
        for (int r0 = 0; r0 < n_rounds; r0 += chunk_trees) {
            const int nc = min(chunk_trees, n_rounds - r0);
            const bool first = r0 == 0, last = r0 + nc >= n_rounds;
            __syncthreads();  // the previous chunk's walks are over
            for (int i = threadIdx.x; i < nc * n_nodes; i += PR_THREADS) {
                const RNode nd = model[((size_t)(r0 + i / n_nodes) * K + t) * n_nodes + i % n_nodes];
                tflags[i] = nd.flags; tweight[i] = nd.weight;
            }
            __syncthreads();
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const unsigned char *rowp[RPT];
                double dsum[RPT];
                float fsum[RPT];
#pragma unroll
                for (int j = 0; j < RPT; ++j) {
                    const int slot = j * PR_THREADS + threadIdx.x;
                    const int i = min(tile * ROWS + slot, n_rows - 1);
                    rowp[j] = bins + (size_t)i * Fpad;
                    if (WORD_ROWS) {  // a thread spreads out its own rows and reads only them back: no barrier needed
                        const uint4 a = reinterpret_cast<const uint4 *>(rowp[j])[0], b = reinterpret_cast<const uint4 *>(rowp[j])[1];
                        words[0 * ROWS + slot] = a.x; words[1 * ROWS + slot] = a.y; words[2 * ROWS + slot] = a.z; words[3 * ROWS + slot] = a.w;
                        words[4 * ROWS + slot] = b.x; words[5 * ROWS + slot] = b.y; words[6 * ROWS + slot] = b.z; words[7 * ROWS + slot] = b.w;
                    }
                    dsum[j] = base_score; fsum[j] = base_score;
                    if (!first) { const double p = partial[(size_t)t * n_rows + i]; dsum[j] = p; fsum[j] = (float)p; }
                }
                for (int c = 0; c < nc; ++c) {
                    const int *ndf = tflags + (size_t)c * n_nodes;
                    const float *ndw = tweight + (size_t)c * n_nodes;
                    int cur[RPT];
#pragma unroll
                    for (int j = 0; j < RPT; ++j) cur[j] = 0;
                    for (int lvl = 0; lvl < depth; ++lvl) {
                        // all rows' node reads first, then their feature reads, then branch-free steps: the walks of a
                        // thread's rows overlap
                        int fl[RPT];
#pragma unroll
                        for (int j = 0; j < RPT; ++j) fl[j] = ndf[cur[j]];
                        uint32_t wd[RPT];
#pragma unroll
                        for (int j = 0; j < RPT; ++j) {
                            const unsigned hi = (unsigned)fl[j] >> 16;
                            if (WORD_ROWS) wd[j] = words[hi * ROWS + j * PR_THREADS + threadIdx.x];
                            else wd[j] = hi < (unsigned)F ? rowp[j][hi] : (unsigned)MISSING_BIN;
                        }
#pragma unroll
                        for (int j = 0; j < RPT; ++j) {
                            const int b = WORD_ROWS ? (int)((wd[j] >> ((fl[j] >> 10) & 31)) & 0xffu) : (int)wd[j];
                            const bool left = (b == MISSING_BIN) ? !(fl[j] & 0x100) : (b <= (fl[j] & 0xff));
                            const int next = 2 * cur[j] + (left ? 1 : 2);
                            cur[j] = (fl[j] & 0x200) ? cur[j] : next;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < RPT; ++j) {
                        const float wt = ndw[cur[j]];
                        if (DENSE_PATH) dsum[j] += (double)__fmul_rn(lr, wt);
                        else fsum[j] = __fmaf_rn(lr, wt, fsum[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < RPT; ++j) {
                    const int i = tile * ROWS + j * PR_THREADS + (int)threadIdx.x;
                    if (i >= n_rows) continue;
                    if (last) out[(size_t)t * n_rows + i] = DENSE_PATH ? (float)(0.0 + dsum[j]) : fsum[j];
                    else partial[(size_t)t * n_rows + i] = DENSE_PATH ? dsum[j] : (double)fsum[j];
                }
            }
        }
    }
}

// ---- traversal on two planes of ranks (rows of at most 32 features) --------------------------------------------------
// The walk above is bound by instruction issue; this one strips the step down to: node (8 bytes), word, byte, compare,
// index.  Three things make that possible.  (1) Every tree is completed to its full depth on the host: below a leaf
// that sits above the last level the nodes pass to the left and the leftmost leaf of the subtree carries the weight,
// so a walk always takes `depth` steps and no step tests for a leaf.  (2) A tile keeps TWO planes of rank words in
// shared memory, the ranks b and the ranks rotated by one, (b + 1) & 255: a node whose missing values go right
// compares b <= t on the first plane (missing = 255 fails), a node whose missing values go left compares
// (b + 1) & 255 <= t + 1 on the second (missing = 0 passes) -- the default direction costs no instruction.
// (3) A node is ONE 32-bit word: the byte-permute selector that moves the feature's byte into the TOP byte of a zero
// word (bits 0-15, used as they are), the index of (plane, word) (16-20) and the threshold in the top byte (24-31):
// `permuted <= node` as unsigned words then IS `byte <= threshold` (the lower 24 bits can only help the right-hand
// side of a tie it already wins), so no field is extracted for the comparison.  ncu: 17.6 warp instructions per row
// and level with fields to extract, issue slots 71 % busy, 1.4 shared-memory wavefronts per read.
typedef unsigned PlaneNode;
__host__ __device__ inline PlaneNode plane_node(unsigned byte, unsigned threshold, unsigned plane_word) {
    return ((byte << 12) | 0x0444u) | (plane_word << 16) | (threshold << 24);
}
constexpr int PL_THREADS = 1024;   // ncu, 512 threads x 4 rows: 4 warps per scheduler, issue slots 60 % busy, stalls on shared-memory
constexpr int PL_RPT = 2;          // reads and on dependent arithmetic: the same tile with twice the warps and half the rows each
constexpr int PL_ROWS = PL_THREADS * PL_RPT;
constexpr int PL_WORDS = 9;  // eight words of a 32-byte row + one word of absent marks per plane

template <bool DENSE_PATH>
__global__ void __launch_bounds__(PL_THREADS)
k_predict_planes(const unsigned char *__restrict__ bins, int Fpad, int n_rows, const PlaneNode *__restrict__ model_nodes,
                 const float *__restrict__ model_leaves, int n_rounds, int K, int depth, int chunk_trees, float lr, float base_score,
                 float *__restrict__ out, double *__restrict__ partial) {
    extern __shared__ __align__(16) unsigned char pl_sm[];
    constexpr int RPT = PL_RPT, ROWS = PL_ROWS;
    uint32_t *words = reinterpret_cast<uint32_t *>(pl_sm);                       // [2][9][ROWS]
    const int n_inner = (1 << depth) - 1, n_leaf = 1 << depth;
    PlaneNode *tnodes = reinterpret_cast<PlaneNode *>(words + 2 * PL_WORDS * ROWS);   // [chunk_trees][n_inner]
    float *tleaves = reinterpret_cast<float *>(tnodes + (size_t)chunk_trees * n_inner);  // [chunk_trees][n_leaf]
    const int n_tiles = (n_rows + ROWS - 1) / ROWS;
    for (int i = threadIdx.x; i < ROWS; i += PL_THREADS) {
        words[(PL_WORDS - 1) * ROWS + i] = 0xffffffffu;         // absent feature: rank 255 ...
        words[(2 * PL_WORDS - 1) * ROWS + i] = 0u;              // ... and its rotation
    }
    for (int t = 0; t < K; ++t) {
        for (int r0 = 0; r0 < n_rounds; r0 += chunk_trees) {
            const int nc = min(chunk_trees, n_rounds - r0);
            const bool first = r0 == 0, last = r0 + nc >= n_rounds;
            __syncthreads();  // the previous chunk's walks are over
            for (int i = threadIdx.x; i < nc * n_inner; i += PL_THREADS)
                tnodes[i] = model_nodes[((size_t)(r0 + i / n_inner) * K + t) * n_inner + i % n_inner];
            for (int i = threadIdx.x; i < nc * n_leaf; i += PL_THREADS)
                tleaves[i] = model_leaves[((size_t)(r0 + i / n_leaf) * K + t) * n_leaf + i % n_leaf];
            __syncthreads();
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                double dsum[RPT];
                float fsum[RPT];
#pragma unroll
                for (int j = 0; j < RPT; ++j) {
                    const int slot = j * PL_THREADS + threadIdx.x;
                    const int i = min(tile * ROWS + slot, n_rows - 1);
                    const uint4 a = reinterpret_cast<const uint4 *>(bins + (size_t)i * Fpad)[0], b = reinterpret_cast<const uint4 *>(bins + (size_t)i * Fpad)[1];
                    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int k = 0; k < 8; ++k) {  // a thread spreads out its own rows and reads only them back: no barrier needed
                        words[k * ROWS + slot] = w[k];
                        words[(PL_WORDS + k) * ROWS + slot] = __vadd4(w[k], 0x01010101u);
                    }
                    dsum[j] = base_score; fsum[j] = base_score;
                    if (!first) { const double p = partial[(size_t)t * n_rows + i]; dsum[j] = p; fsum[j] = (float)p; }
                }
                for (int c = 0; c < nc; ++c) {
                    const PlaneNode *nd = tnodes + (size_t)c * n_inner;
                    unsigned cur[RPT];
#pragma unroll
                    for (int j = 0; j < RPT; ++j) cur[j] = 0;
                    auto level = [&]() {
                        PlaneNode n[RPT];
#pragma unroll
                        for (int j = 0; j < RPT; ++j) n[j] = nd[cur[j]];
                        uint32_t w[RPT];
#pragma unroll
                        for (int j = 0; j < RPT; ++j)   // [(plane, word)][row slot]
                            w[j] = words[((n[j] >> 16) & 0xffu) * (unsigned)ROWS + (unsigned)(j * PL_THREADS) + threadIdx.x];
#pragma unroll
                        for (int j = 0; j < RPT; ++j)
                            cur[j] = 2 * cur[j] + (__byte_perm(w[j], 0u, n[j]) <= n[j] ? 1 : 2);
                    };
                    if (depth == 8) {   // the usual depth, unrolled
#pragma unroll
                        for (int lvl = 0; lvl < 8; ++lvl) level();
                    } else {
#pragma unroll 1
                        for (int lvl = 0; lvl < depth; ++lvl) level();
                    }
                    const float *lw = tleaves + (size_t)c * n_leaf - n_inner;
#pragma unroll
                    for (int j = 0; j < RPT; ++j) {
                        const float wt = lw[cur[j]];
                        if (DENSE_PATH) dsum[j] += (double)__fmul_rn(lr, wt);
                        else fsum[j] = __fmaf_rn(lr, wt, fsum[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < RPT; ++j) {
                    const int i = tile * ROWS + j * PL_THREADS + (int)threadIdx.x;
                    if (i >= n_rows) continue;
                    if (last) out[(size_t)t * n_rows + i] = DENSE_PATH ? (float)(0.0 + dsum[j]) : fsum[j];
                    else partial[(size_t)t * n_rows + i] = DENSE_PATH ? dsum[j] : (double)fsum[j];
                }
            }
        }
    }
}

void predict_raw(const DataSet &ds, const std::vector<std::vector<Tree>> &model, float learning_rate, float base_score,
                 std::vector<float> &out, float *kernel_ms) {
    const int N = ds.n_rows;
    const int n_rounds = (int)model.size();
    TGBM_CHECK(n_rounds > 0 && !model[0].empty(), "empty model");
    const int K = (int)model[0].size();
    const int n_nodes = (int)model[0][0].nodes.size();
    out.assign((size_t)N * K, 0.f);
    if (N == 0) return;
    if (K > 1) base_score = 0;  // predictor.cu:81-83
    std::vector<PNode> flat((size_t)n_rounds * K * n_nodes);
    for (int r = 0; r < n_rounds; ++r)
        for (int t = 0; t < K; ++t) {
            TGBM_CHECK((int)model[r].size() == K && (int)model[r][t].nodes.size() == n_nodes, "ragged model");
            for (int n = 0; n < n_nodes; ++n) {
                const TreeNode &s = model[r][t].nodes[n];
                PNode &d = flat[((size_t)r * K + t) * n_nodes + n];
                d.lch = s.lch_index; d.rch = s.rch_index;
                if (s.is_leaf) { d.v = s.base_weight; d.fid = (int)0x80000000; }
                else { d.v = s.split_value; d.fid = (s.split_feature_id & 0x3fffffff) | (s.default_right ? 0x40000000 : 0); }
            }
        }
    // is every tree a heap (children of i at 2i+1, 2i+2)?  The trainers here and the reference's Tree::init2 build them so.
    bool heap = ((n_nodes + 1) & n_nodes) == 0;
    int depth = 0;
    while ((2 << depth) - 1 < n_nodes) ++depth;
    std::vector<HNode> hflat;
    if (heap) {
        hflat.resize(flat.size());
        for (size_t i = 0; i < flat.size() && heap; ++i) {
            const int n = (int)(i % n_nodes);
            const PNode &s = flat[i];
            if (!(s.fid & 0x80000000) && (s.lch != 2 * n + 1 || s.rch != 2 * n + 2 || s.rch >= n_nodes)) heap = false;
            hflat[i].v = s.v;
            hflat[i].fid = s.fid;
        }
    }
    // streams and events are released on every way out, also when a CUDA call throws
    struct Guard {
        cudaStream_t st = nullptr;
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        ~Guard() {
            if (e0) cudaEventDestroy(e0);
            if (e1) cudaEventDestroy(e1);
            if (st) cudaStreamDestroy(st);
        }
    } gd;
    TGBM_CUDA(cudaStreamCreateWithFlags(&gd.st, cudaStreamNonBlocking));
    cudaStream_t st = gd.st;
    const size_t nnz = (size_t)ds.rp[N];
    DevBuf<int> d_rp, d_col;
    DevBuf<float> d_val, d_out;
    DevBuf<PNode> d_model;
    DevBuf<HNode> d_hmodel;
    d_rp.alloc(N + 1); d_col.alloc(std::max<size_t>(nnz, 1)); d_val.alloc(std::max<size_t>(nnz, 1)); d_out.alloc((size_t)N * K);
    upload_h2d(d_rp.p, ds.rp, sizeof(int) * (size_t)(N + 1), st, upload_threads());
    upload_h2d(d_col.p, ds.ci, sizeof(int) * nnz, st, upload_threads());
    upload_h2d(d_val.p, ds.vv, sizeof(float) * nnz, st, upload_threads());
    if (heap) {
        d_hmodel.alloc(hflat.size());
        TGBM_CUDA(cudaMemcpyAsync(d_hmodel.p, hflat.data(), sizeof(HNode) * hflat.size(), cudaMemcpyHostToDevice, st));
    }
    d_model.alloc(flat.size());
    TGBM_CUDA(cudaMemcpyAsync(d_model.p, flat.data(), sizeof(PNode) * flat.size(), cudaMemcpyHostToDevice, st));
    const int F = ds.n_features;
    const size_t smem = (size_t)F * PRED_ROWS * sizeof(float);
    int dev = 0, num_sms = 148;
    TGBM_CUDA(cudaGetDevice(&dev));
    TGBM_CUDA(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
    // The reference chooses its arithmetic by F * 128 * 4 <= 48 KB (predictor.cu:88); that choice is kept, the tiled
    // kernel serves either whenever a tile of rows and a chunk of trees fit the shared memory of an SM.
    const bool dense_path = smem <= 48 * 1024;
    bool done = false;
    DevBuf<double> d_partial;
    const bool heap_ok = heap && getenv("TGBM_PREDICT_SIMPLE") == nullptr;
    // ---- ranks: thresholds per feature, nodes with threshold ranks
    std::vector<int> thr_ptr;
    std::vector<float> thr;
    std::vector<RNode> rflat;
    // (the rank bytes are a dense N x Fpad matrix: not for wide sparse data, where it would dwarf the CSR itself)
    const size_t rank_bytes = (size_t)N * (size_t)((F + 31) / 32 * 32);
    bool ranks = heap_ok && getenv("TGBM_PREDICT_FLOAT") == nullptr && sizeof(RNode) * (size_t)n_nodes * std::min(8, n_rounds) <= 140 * 1024 && F < 65536 &&
                 rank_bytes <= std::max<size_t>((size_t)64 << 20, 8 * nnz);
    if (ranks) {
        std::vector<std::vector<float>> per(F);
        for (size_t i = 0; i < flat.size(); ++i) {
            const PNode &nd = flat[i];
            if (nd.fid & 0x80000000) continue;
            const int f = nd.fid & 0x3fffffff;
            if (f < F) per[f].push_back(nd.v == 0.f ? 0.f : nd.v);  // -0 and +0 compare equal: one threshold
            if (nd.v != nd.v) ranks = false;                        // a NaN threshold has no rank
        }
        thr_ptr.assign(F + 1, 0);
        for (int f = 0; f < F && ranks; ++f) {
            std::sort(per[f].begin(), per[f].end());
            per[f].erase(std::unique(per[f].begin(), per[f].end()), per[f].end());
            if (per[f].size() > 254) ranks = false;
            thr_ptr[f + 1] = thr_ptr[f] + (int)per[f].size();
        }
        if (ranks) {
            thr.reserve(thr_ptr[F] + 1);
            for (int f = 0; f < F; ++f) thr.insert(thr.end(), per[f].begin(), per[f].end());
            rflat.resize(flat.size());
            for (size_t i = 0; i < flat.size(); ++i) {
                const PNode &nd = flat[i];
                RNode &o = rflat[i];
                if (nd.fid & 0x80000000) { o.flags = 0x200; o.weight = nd.v; continue; }
                const int f = nd.fid & 0x3fffffff;
                int t = 0;
                if (f < F) t = (int)(std::lower_bound(per[f].begin(), per[f].end(), nd.v == 0.f ? 0.f : nd.v) - per[f].begin());
                // rows of up to 32 features are walked on words: bits 16-31 = word index (8 = the word of absent marks, for a
                // feature the data does not have), bits 10-14 = bit offset of the byte; else bits 16-31 = feature id
                const unsigned hi = (F <= 32) ? (f < F ? (unsigned)(f >> 2) : 8u) : (unsigned)std::min(f, 65535);
                o.flags = t | ((nd.fid & 0x40000000) ? 0x100 : 0) | ((F <= 32 && f < F) ? ((f & 3) * 8) << 10 : 0) | (int)(hi << 16);
                o.weight = 0.f;
            }
        }
    }
    // complete trees for the two-plane walk (rows of at most 32 features; TGBM_PREDICT_RANKS=1 keeps the walk above)
    const bool planes = ranks && F <= 32 && depth >= 1 && depth <= 12 && getenv("TGBM_PREDICT_RANKS") == nullptr;
    std::vector<PlaneNode> pl_nodes;
    std::vector<float> pl_leaves;
    const int n_inner = (1 << depth) - 1, n_leaf = 1 << depth;
    if (planes) {
        pl_nodes.resize((size_t)n_rounds * K * n_inner);
        pl_leaves.assign((size_t)n_rounds * K * n_leaf, 0.f);
        const PlaneNode pass = plane_node(0, 255, PL_WORDS - 1);   // absent word of plane 0: 255 <= 255, left
        for (int tr = 0; tr < n_rounds * K; ++tr) {
            const RNode *src = rflat.data() + (size_t)tr * n_nodes;
            PlaneNode *dn = pl_nodes.data() + (size_t)tr * n_inner;
            float *dl = pl_leaves.data() + (size_t)tr * n_leaf;
            // carry[i]: the node inherits a leaf from above (1) with weight w[i], or lies off every path (2)
            std::vector<unsigned char> carry(n_nodes, 0);
            std::vector<float> w(n_nodes, 0.f);
            for (int i = 0; i < n_nodes; ++i) {
                const bool leaf = carry[i] != 0 || (src[i].flags & 0x200);
                const float wt = carry[i] == 1 ? w[i] : carry[i] == 2 ? 0.f : src[i].weight;
                if (i >= n_inner) { dl[i - n_inner] = leaf ? wt : 0.f; continue; }
                if (leaf) {
                    dn[i] = pass;
                    carry[2 * i + 1] = carry[i] == 2 ? 2 : 1; w[2 * i + 1] = wt;
                    carry[2 * i + 2] = 2;
                    continue;
                }
                const int fl = src[i].flags;
                const unsigned word = (unsigned)fl >> 16, byte = (((unsigned)fl >> 10) & 31u) / 8u, t = (unsigned)fl & 0xffu;
                const bool default_right = fl & 0x100;
                // missing goes right: plane 0, rank <= t; missing goes left: plane 1 (ranks rotated by one), <= t + 1
                dn[i] = plane_node(byte, default_right ? t : t + 1, word + (default_right ? 0u : (unsigned)PL_WORDS));
            }
        }
    }
    DevBuf<PlaneNode> d_pl_nodes;
    DevBuf<float> d_pl_leaves;
    DevBuf<int> d_thr_ptr;
    DevBuf<float> d_thr;
    DevBuf<RNode> d_rmodel;
    DevBuf<unsigned char> d_bins;
    const int Fpad = (F + 31) / 32 * 32;
    int rk_chunk = 0;
    if (ranks) {
        d_thr_ptr.alloc(F + 1); d_thr.alloc(std::max<size_t>(thr.size(), 1)); d_rmodel.alloc(rflat.size()); d_bins.alloc((size_t)N * Fpad);
        TGBM_CUDA(cudaMemcpyAsync(d_thr_ptr.p, thr_ptr.data(), sizeof(int) * (F + 1), cudaMemcpyHostToDevice, st));
        if (!thr.empty()) TGBM_CUDA(cudaMemcpyAsync(d_thr.p, thr.data(), sizeof(float) * thr.size(), cudaMemcpyHostToDevice, st));
        TGBM_CUDA(cudaMemcpyAsync(d_rmodel.p, rflat.data(), sizeof(RNode) * rflat.size(), cudaMemcpyHostToDevice, st));
        const size_t rk_rows_bytes = F <= 32 ? sizeof(uint32_t) * 9 * PR_ROWS : 0;
        rk_chunk = (int)std::min<size_t>((size_t)n_rounds, ((size_t)(216 * 1024) - rk_rows_bytes) / (sizeof(RNode) * (size_t)n_nodes));
        if (planes) {
            d_pl_nodes.alloc(pl_nodes.size()); d_pl_leaves.alloc(pl_leaves.size());
            TGBM_CUDA(cudaMemcpyAsync(d_pl_nodes.p, pl_nodes.data(), sizeof(PlaneNode) * pl_nodes.size(), cudaMemcpyHostToDevice, st));
            TGBM_CUDA(cudaMemcpyAsync(d_pl_leaves.p, pl_leaves.data(), sizeof(float) * pl_leaves.size(), cudaMemcpyHostToDevice, st));
            const size_t per_tree = sizeof(PlaneNode) * (size_t)n_inner + sizeof(float) * (size_t)n_leaf;
            const size_t row_bytes = sizeof(uint32_t) * 2 * PL_WORDS * PL_ROWS;
            rk_chunk = (int)std::min<size_t>((size_t)n_rounds, ((size_t)(224 * 1024) - row_bytes) / per_tree);
            TGBM_CHECK(rk_chunk >= 1, "a tree of this depth does not fit beside a tile of rows");
        }
        if (rk_chunk < n_rounds) d_partial.alloc((size_t)N * K);
    }
    const bool tiled = heap_ok && !ranks;
    auto tiles = [&](bool plan_only) {
        return dense_path ? launch_predict_tiles<true>(d_rp.p, d_col.p, d_val.p, N, F, d_hmodel.p, n_rounds, K, n_nodes, depth, learning_rate,
                                                       base_score, d_out.p, num_sms, st, d_partial, plan_only)
                          : launch_predict_tiles<false>(d_rp.p, d_col.p, d_val.p, N, F, d_hmodel.p, n_rounds, K, n_nodes, depth, learning_rate,
                                                        base_score, d_out.p, num_sms, st, d_partial, plan_only);
    };
    if (tiled) tiles(true);  // scratch for the running sums is allocated here, outside the timed kernel
    // dense fast path of the conversion: N * F stored values, F a multiple of 4 up to 32
    bool dense_rows = ranks && planes && F % 4 == 0 && (size_t)N * F == nnz && getenv("TGBM_PREDICT_RANKS") == nullptr;
    // (whether row i really starts at i * F and holds the columns 0 .. F-1 is checked by the kernel, row by row)
    DevBuf<float> d_tree_thr;
    DevBuf<int> d_not_dense;
    if (dense_rows) {
        std::vector<float> tree((size_t)F * 256, INFINITY);
        for (int f = 0; f < F; ++f) {
            std::vector<float> sorted(255, INFINITY);
            std::copy(thr.begin() + thr_ptr[f], thr.begin() + thr_ptr[f + 1], sorted.begin());
            // node k of the implicit tree holds the middle of its range; children 2k+1 (left half), 2k+2 (right half)
            struct Range { int k, lo, hi; };
            std::vector<Range> todo{{0, 0, 255}};
            while (!todo.empty()) {
                const Range g = todo.back();
                todo.pop_back();
                if (g.lo >= g.hi) continue;
                const int mid = (g.lo + g.hi) / 2;
                tree[(size_t)f * 256 + g.k] = sorted[mid];
                todo.push_back({2 * g.k + 1, g.lo, mid});
                todo.push_back({2 * g.k + 2, mid + 1, g.hi});
            }
        }
        d_tree_thr.alloc(tree.size()); d_not_dense.alloc(1);
        TGBM_CUDA(cudaMemcpyAsync(d_tree_thr.p, tree.data(), sizeof(float) * tree.size(), cudaMemcpyHostToDevice, st));
        d_not_dense.zero(st);
    }
    if (ranks) {   // the kernels of this path are loaded before the clock starts (the first launch of a kernel loads it otherwise)
        cudaFuncAttributes fa;
        if (dense_rows) cudaFuncGetAttributes(&fa, dense_path ? k_rank_dense_rows<true> : k_rank_dense_rows<false>);
        cudaFuncGetAttributes(&fa, dense_path ? k_rank_rows<true, true> : k_rank_rows<false, true>);
        if (planes) cudaFuncGetAttributes(&fa, dense_path ? k_predict_planes<true> : k_predict_planes<false>);
    }
    if (kernel_ms) { TGBM_CUDA(cudaEventCreate(&gd.e0)); TGBM_CUDA(cudaEventCreate(&gd.e1)); TGBM_CUDA(cudaEventRecord(gd.e0, st)); }
    if (tiled) done = tiles(false);
    if (ranks) {
        bool converted = false;
        if (dense_rows) {
            const size_t tree_smem = sizeof(float) * (size_t)F * 256;
            auto kern = dense_path ? k_rank_dense_rows<true> : k_rank_dense_rows<false>;
            kern<<<std::min((N + RD_THREADS - 1) / RD_THREADS, num_sms * 8), RD_THREADS, tree_smem, st>>>(d_rp.p, d_col.p, d_val.p, N, F, d_tree_thr.p,
                                                                                                      d_thr_ptr.p, d_bins.p, d_not_dense.p);
            int h_not_dense = 0;
            TGBM_CUDA(cudaMemcpyAsync(&h_not_dense, d_not_dense.p, sizeof(int), cudaMemcpyDeviceToHost, st));
            TGBM_CUDA(cudaStreamSynchronize(st));
            converted = h_not_dense == 0;
        }
        if (!converted) {
        TGBM_CUDA(cudaMemsetAsync(d_bins.p, MISSING_BIN, d_bins.bytes(), st));
        const int rk_blocks = std::min((N + RK_ROWS - 1) / RK_ROWS, num_sms * 8);   // persistent: a block walks several tiles of rows
        const size_t thr_smem = sizeof(float) * (size_t)F * RK_THR_STRIDE;
        const bool smem_thr = thr_smem <= 40 * 1024 && getenv("TGBM_PREDICT_RANKS") == nullptr;
        if (smem_thr) {
            if (dense_path) k_rank_rows<true, true><<<rk_blocks, RK_THREADS, thr_smem, st>>>(d_rp.p, d_col.p, d_val.p, N, F, Fpad, d_thr_ptr.p, d_thr.p, d_bins.p);
            else k_rank_rows<false, true><<<rk_blocks, RK_THREADS, thr_smem, st>>>(d_rp.p, d_col.p, d_val.p, N, F, Fpad, d_thr_ptr.p, d_thr.p, d_bins.p);
        } else {
            if (dense_path) k_rank_rows<true, false><<<rk_blocks, RK_THREADS, 0, st>>>(d_rp.p, d_col.p, d_val.p, N, F, Fpad, d_thr_ptr.p, d_thr.p, d_bins.p);
            else k_rank_rows<false, false><<<rk_blocks, RK_THREADS, 0, st>>>(d_rp.p, d_col.p, d_val.p, N, F, Fpad, d_thr_ptr.p, d_thr.p, d_bins.p);
        }
        }
        const size_t rk_smem = sizeof(RNode) * (size_t)n_nodes * rk_chunk + (F <= 32 ? sizeof(uint32_t) * 9 * PR_ROWS : 0);
        const int grid = std::max(1, std::min((N + PR_ROWS - 1) / PR_ROWS, num_sms));
        if (getenv("TGBM_TIMING")) {  // how the time splits between the conversion and the walk
            cudaEvent_t em;
            cudaEventCreate(&em); cudaEventRecord(em, st); cudaEventSynchronize(em);
            float ms = 0;
            if (gd.e0) { cudaEventElapsedTime(&ms, gd.e0, em); fprintf(stderr, "[tgbm predict] rows -> ranks %8.3f ms\n", ms); }
            cudaEventDestroy(em);
        }
        auto go = [&](auto kern) {
            TGBM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rk_smem));
            kern<<<grid, PR_THREADS, rk_smem, st>>>(d_bins.p, Fpad, F, N, d_rmodel.p, n_rounds, K, n_nodes, depth, rk_chunk, learning_rate, base_score,
                                             d_out.p, d_partial.p);
        };
        if (planes) {
            const size_t pl_smem = sizeof(uint32_t) * 2 * PL_WORDS * PL_ROWS +
                                   (sizeof(PlaneNode) * (size_t)n_inner + sizeof(float) * (size_t)n_leaf) * rk_chunk;
            const int pl_grid = std::max(1, std::min((N + PL_ROWS - 1) / PL_ROWS, num_sms));
            auto go_planes = [&](auto kern) {
                TGBM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl_smem));
                kern<<<pl_grid, PL_THREADS, pl_smem, st>>>(d_bins.p, Fpad, N, d_pl_nodes.p, d_pl_leaves.p, n_rounds, K, depth, rk_chunk, learning_rate,
                                                          base_score, d_out.p, d_partial.p);
            };
            if (dense_path) go_planes(k_predict_planes<true>); else go_planes(k_predict_planes<false>);
        }
        else if (dense_path) { if (F <= 32) go(k_predict_ranks<true, true>); else go(k_predict_ranks<true, false>); }
        else { if (F <= 32) go(k_predict_ranks<false, true>); else go(k_predict_ranks<false, false>); }
        done = true;
    }
    if (done) {
    } else if (dense_path) {
        k_predict_dense<<<(N + PRED_ROWS - 1) / PRED_ROWS, PRED_ROWS, smem, st>>>(d_rp.p, d_col.p, d_val.p, N, F, d_model.p, n_rounds, K,
                                                                                n_nodes, learning_rate, base_score, d_out.p);
    } else if (smem <= 200 * 1024) {
        TGBM_CUDA(cudaFuncSetAttribute(k_predict_csr_staged, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k_predict_csr_staged<<<(N + PRED_ROWS - 1) / PRED_ROWS, PRED_ROWS, smem, st>>>(d_rp.p, d_col.p, d_val.p, N, F, d_model.p, n_rounds,
                                                                                     K, n_nodes, learning_rate, base_score, d_out.p);
    } else {
        k_predict_csr<<<(N + 127) / 128, 128, 0, st>>>(d_rp.p, d_col.p, d_val.p, N, d_model.p, n_rounds, K, n_nodes, learning_rate,
                                                       base_score, d_out.p);
    }
    TGBM_CUDA(cudaGetLastError());
    if (kernel_ms) TGBM_CUDA(cudaEventRecord(gd.e1, st));
    TGBM_CUDA(cudaMemcpyAsync(out.data(), d_out.p, sizeof(float) * out.size(), cudaMemcpyDeviceToHost, st));
    TGBM_CUDA(cudaStreamSynchronize(st));
    if (kernel_ms) TGBM_CUDA(cudaEventElapsedTime(kernel_ms, gd.e0, gd.e1));
}

// ---- predict_transform -------------------------------------------------------------------------
// regression_obj.h:27-32 (identity / sigmoid), :76-92 (binary: label[y > 0]),
// multiclass_obj.cu:44-89 (softmax: label of the arg max; softprob: probabilities, class-major)
__global__ void k_transform(int objective, int K, int n, const float *__restrict__ label, float *__restrict__ y) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (objective == REG_LOGISTIC) {
        y[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, portable_expf(-y[i])));
    } else if (objective == BINARY_LOGISTIC) {
        y[i] = label[y[i] > 0.f ? 1 : 0];
    } else if (objective == MULTI_SOFTMAX) {
        int mk = 0;
        float mp = y[i];
        for (int k = 1; k < K; ++k) if (mp < y[(size_t)k * n + i]) { mp = y[(size_t)k * n + i]; mk = k; }
        y[i] = label[mk];
    } else if (objective == MULTI_SOFTPROB) {
        float mx = y[i];
        for (int k = 1; k < K; ++k) mx = fmaxf(mx, y[(size_t)k * n + i]);
        float sum = 0.f;
        for (int k = 0; k < K; ++k) {
            const float e = portable_expf(__fsub_rn(y[(size_t)k * n + i], mx));
            y[(size_t)k * n + i] = e;
            sum = __fadd_rn(sum, e);
        }
        for (int k = 0; k < K; ++k) y[(size_t)k * n + i] = __fdiv_rn(y[(size_t)k * n + i], sum);
    }
}

void predict_transform(int objective, int num_class, const std::vector<float> &label, int n_rows, std::vector<float> &y) {
    if (objective == REG_LINEAR || objective == RANK_PAIRWISE || objective == RANK_NDCG || n_rows == 0) return;
    int K = (int)(y.size() / (size_t)n_rows);
    if (objective == BINARY_LOGISTIC) TGBM_CHECK(label.size() >= 2, "binary:logistic needs two class labels");
    if (objective == MULTI_SOFTMAX) TGBM_CHECK((int)label.size() >= K, "multi:softmax needs one label per class");
    (void)num_class;
    DevBuf<float> d_y, d_label;
    d_y.alloc(y.size()); d_label.alloc(std::max<size_t>(label.size(), 1));
    TGBM_CUDA(cudaMemcpy(d_y.p, y.data(), sizeof(float) * y.size(), cudaMemcpyHostToDevice));
    if (!label.empty()) TGBM_CUDA(cudaMemcpy(d_label.p, label.data(), sizeof(float) * label.size(), cudaMemcpyHostToDevice));
    k_transform<<<(n_rows + 255) / 256, 256>>>(objective, K, n_rows, d_label.p, d_y.p);
    TGBM_CUDA(cudaGetLastError());
    if (objective == MULTI_SOFTMAX) y.resize(n_rows);
    TGBM_CUDA(cudaMemcpy(y.data(), d_y.p, sizeof(float) * y.size(), cudaMemcpyDeviceToHost));
}

// ---- metric on raw scores (Predictor::predict logs it, predictor.cu:20-24) ---------------------
float metric_score(int objective, const DataSet &ds, int num_class, const std::vector<float> &raw) {
    const int N = ds.n_rows;
    if (N == 0) return 0.f;
    const int K = (int)(raw.size() / (size_t)N);
    (void)num_class;
    DevBuf<float> d_y, d_raw, d_out;
    d_y.alloc(N); d_raw.alloc(raw.size()); d_out.alloc(1);
    TGBM_CUDA(cudaMemcpy(d_y.p, ds.yv ? ds.yv : ds.y.data(), sizeof(float) * N, cudaMemcpyHostToDevice));
    TGBM_CUDA(cudaMemcpy(d_raw.p, raw.data(), sizeof(float) * raw.size(), cudaMemcpyHostToDevice));
    if (need_group_file(objective)) {
        RankState rs;
        rs.init(ds, objective, N, nullptr, 0, (long long)ds.group.size());
        rs.metric(objective, d_raw.p, d_out.p, nullptr, N, nullptr);
    } else {
        DevBuf<double> partial, sum;
        const int blocks = std::max(1, std::min((N + 255) / 256, 1024));
        partial.alloc(blocks); sum.alloc(1);
        k_metric_partial<<<blocks, 256>>>(objective, d_y.p, d_raw.p, N, K, partial.p);
        k_metric_sum<<<1, 32>>>(partial.p, blocks, sum.p);
        k_metric_final<<<1, 32>>>(objective, sum.p, N, d_out.p);
    }
    TGBM_CUDA(cudaGetLastError());
    float r = 0;
    TGBM_CUDA(cudaMemcpy(&r, d_out.p, sizeof(float), cudaMemcpyDeviceToHost));
    return r;
}

}  // namespace tgbm
