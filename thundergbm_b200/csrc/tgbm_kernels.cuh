// CUDA kernels of the histogram tree builder (sm_100a).
//
// Data layout in HBM (one rank = one contiguous block of rows):
//   bins   uint8 [N][Fpad]   row-major local bin ids, Fpad = F rounded up to 32, 255 = missing.
//                            One 32-byte sector holds 32 features of one row.
//   binsT  uint8 [F][Npad]   the same matrix column-major; read by the partition step, which
//                            needs one feature of many rows.
//   gh     float2 [K][N]     gradient pairs of the round, class-major like the reference.
//   ghq    int2   [K][N]     the same on the round's fixed-point grid.
//   rec_idx/rec_gh [2][N]    per-level record lists: rows grouped by tree node, ascending row id
//                            inside a node (stable partition), ping-pong between levels.
//   hist   int64 [node][B][2] per-node histograms on the fixed-point grid.
//
// All sums on the fixed-point grid are integer sums, so they do not depend on the order of
// the atomics, on the CTA count or on the number of ranks.
#pragma once
#include "tgbm_device.cuh"

namespace tgbm {

constexpr int HIST_THREADS = 1024;  // one CTA per SM: 64 KB of int32 accumulators + up to 128 KB of int64 totals
constexpr int PART_THREADS = 512;  // 512 x 4 records per tile measured best (1024: fewer tiles in flight per SM, 256: longer tile scan)
constexpr int PART_RPT = 4;         // records per thread
constexpr int PART_TILE = PART_THREADS * PART_RPT;
constexpr int MISSING_BIN = 255;

struct HistWork {  // one histogram to build at a level
    int begin, count, slab;
    int vk;  // dense layout: first share (bits 0-15) and number of shares (bits 16-31) of the item, see hist_sequence
};
// Shares of the level's tiles per CTA of the dense histogram kernel.  More shares balance the CTAs better but widen the
// window of rows the GPU works on at a time; 1 to 4 measure the same on 10.5 M rows, 16 is 10 % slower.
constexpr int HIST_SHARES = 2;
constexpr int HIST_MAX_CTAS = 256;  // grid.x limit of the dense histogram kernel (one CTA per SM)

// Device copy of the booster's round counter: kernels whose work depends on the round read it here, so that the launch
// sequence of a round is the same every round and can be replayed as a CUDA graph.
struct RoundState {
    int round;
};

struct TreeCtl {  // device-side scalars of the tree being built
    int n_hist_tiles;
    int n_hist_work;
    int n_part_tiles[2];  // by level parity: level l+1 is planned while level l is still being scattered
    int n_records;  // records alive at the current level
    unsigned long long stat_rows_root, stat_rows_gather, stat_hists, stat_part_rows;
    // single-pass partition: next tile to hand out, tag of the running pass in the tile status words, and a word the
    // host reads after a sync: non-zero when a bounded wait gave up (1 + the tile that waited)
    int part_ticket;
    unsigned part_epoch;
    int error;
};

struct SplitRec {  // best candidate of one (node, feature)
    float gain;     // signed like the reference: negative = missing goes right
    int bin;        // local bin of the candidate, -1 = none
    float lg, lh;   // left sum without missing
    float mg, mh;   // missing sum of the feature in this node
};

// ------------------------------------------------------------------ cut points
// key = feature id in the high word, order-preserving image of the float in the low word
static __global__ void k_make_keys(const float *__restrict__ val, const int *__restrict__ col, size_t nnz,
                            unsigned long long *__restrict__ keys) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nnz; i += (size_t)gridDim.x * blockDim.x) {
        unsigned u = __float_as_uint(val[i]);
        if (u == 0x80000000u) u = 0;  // -0.0f == 0.0f
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        keys[i] = ((unsigned long long)(unsigned)col[i] << 32) | u;
    }
}

__device__ inline float key_to_float(unsigned long long k) {
    unsigned u = (unsigned)(k & 0xffffffffull);
    u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    return __uint_as_float(u);
}

// ustart[f] = number of unique (feature,value) keys with feature < f
static __global__ void k_feature_bounds(const unsigned long long *__restrict__ ukeys, long long nu, int F, long long *__restrict__ ustart) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f > F) return;
    const unsigned long long target = (unsigned long long)(unsigned)f << 32;
    long long lo = 0, hi = nu;
    while (lo < hi) {
        const long long mid = lo + (hi - lo) / 2;
        if (ukeys[mid] < target) lo = mid + 1; else hi = mid;
    }
    ustart[f] = lo;
}

// HistCut::get_cut_points_single (src/thundergbm/hist_cut.cu:232-286): stride s = u / max_bin;
// s == 0 keeps every distinct value, else positions 0, s, ..., (max_bin-1) s
static __global__ void k_select_cuts(const unsigned long long *__restrict__ ukeys, long long nu, const long long *__restrict__ ustart,
                              const int *__restrict__ stride, const int *__restrict__ cut_ptr, int max_bin,
                              float *__restrict__ cut_val, int *__restrict__ cut_fid, int down) {
    // down: the keys carry the complement of the float's ordered image (candidates of the column-sharded builder,
    // largest value first)
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nu; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long k = ukeys[i];
        const int f = (int)(k >> 32);
        const long long t = i - ustart[f];
        const int s = stride[f];
        long long pos;
        if (s == 0) pos = t;
        else if (t % s == 0 && t / s < max_bin) pos = t / s;
        else continue;
        cut_val[cut_ptr[f] + pos] = key_to_float(down ? (k ^ 0xffffffffull) : k);
        cut_fid[cut_ptr[f] + pos] = f;
    }
}

// ------------------------------------------------------------------ cut points of the column-sharded builder
// HistCut::get_cut_points3 + unique_by_flag (src/thundergbm/hist_cut.cu:104-187), which every device of the
// reference runs on its own block of columns: each stored value v of local column j becomes t = v + j*(m+1), m the
// largest value on the device; all t of the device are sorted descending; the column ids are laid over the sorted
// array by COUNT, largest id first; runs of equal t keep their first entry; t goes back to t - j*(m+1) with the id
// found there.  Done here on the distinct (feature, value) keys with their multiplicities: the position of a key's
// first copy in the reference's sorted array is the number of copies before it.
struct ColumnShift {            // per feature
    int shard, first;           // device that owns it in the reference, first column of that device
    float step;                 // m + 1 of that device
    long long below;            // copies in the device's columns with a LARGER id: where this column's ids start
};
__device__ __forceinline__ unsigned float_order(float v) {
    unsigned u = __float_as_uint(v);
    if (u == 0x80000000u) u = 0;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float order_float(unsigned u) {
    u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    return __uint_as_float(u);
}
// key (feature, value) -> (device, complement of the ordered image of t): ascending keys = descending t per device
static __global__ void k_shift_keys(const unsigned long long *__restrict__ ukeys, long long nu, const ColumnShift *__restrict__ cs,
                                    unsigned long long *__restrict__ out) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nu; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long k = ukeys[i];
        const int f = (int)(k >> 32);
        const ColumnShift c = cs[f];
        const float v = key_to_float(k), j = (float)(f - c.first);
        const float t = __fmaf_rn(j, c.step, v);  // one rounding: what nvcc makes of the reference's `v + j * step`
        out[i] = ((unsigned long long)(unsigned)c.shard << 32) | (unsigned)~float_order(t);
    }
}
// sorted shifted keys + the number of copies before each -> candidate keys (feature, complement of the ordered image of
// the value shifted back), all-ones for the entries that unique_by_key drops
static __global__ void k_unshift_keys(const unsigned long long *__restrict__ skeys, const long long *__restrict__ before, long long nu,
                                      const ColumnShift *__restrict__ cs, const int *__restrict__ shard_first,
                                      const int *__restrict__ shard_cols, const long long *__restrict__ shard_before,
                                      unsigned long long *__restrict__ out, unsigned long long *__restrict__ n_heads) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nu; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long k = skeys[i];
        if (i > 0 && skeys[i - 1] == k) { out[i] = ~0ull; continue; }
        const int d = (int)(k >> 32), first = shard_first[d];
        const long long pos = before[i] - shard_before[d];
        int lo = 0, hi = shard_cols[d] - 1;  // smallest local id whose ids start at or before pos (`below` falls as the id grows)
        while (lo < hi) {
            const int mid = (lo + hi) / 2;
            if (cs[first + mid].below <= pos) hi = mid; else lo = mid + 1;
        }
        const float t = order_float(~(unsigned)(k & 0xffffffffull)), j = (float)lo, step = cs[first + lo].step;
        const float v = __fmaf_rn(-j, step, t);
        out[i] = ((unsigned long long)(unsigned)(first + lo) << 32) | (unsigned)~float_order(v);
        atomicAdd(n_heads, 1ull);
    }
}
static __global__ void k_fill_ll(long long *p, size_t n, long long v) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}
// per feature: largest stored value (the last of its ascending keys) and the number of copies before its first key
static __global__ void k_feature_max_before(const unsigned long long *__restrict__ ukeys, const long long *__restrict__ ustart,
                                            const long long *__restrict__ before, long long nu, long long total, int F,
                                            float *__restrict__ fmax, long long *__restrict__ fbefore) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f > F) return;
    const long long a = ustart[f];
    fbefore[f] = a < nu ? before[a] : total;
    if (f < F) fmax[f] = ustart[f + 1] > a ? key_to_float(ukeys[ustart[f + 1] - 1]) : -INFINITY;
}

// HistTreeBuilder::get_bin_ids of the column-sharded builder (hist_tree_builder.cu:31-49): the cut points of a
// feature descend there; first position in [lo, hi] whose cut is <= v, hi when there is none
__device__ __forceinline__ int bin_search_down(const float *__restrict__ cut_val, int lo, int hi, float v) {
    while (lo != hi) {
        const int mid = lo + (hi - lo) / 2;
        if (cut_val[mid] <= v) hi = mid; else lo = mid + 1;
    }
    return lo;
}

// HistTreeBuilder_single::get_bin_ids (hist_tree_builder_single.cu:81-119): clamped upper bound,
// bin = min(#cuts <= v, n_cuts - 1); stored as the feature-local id in both layouts
static __global__ void k_bin_dense(const int *__restrict__ row_ptr, const int *__restrict__ col, const float *__restrict__ val,
                            int n_rows, const int *__restrict__ cut_ptr, const float *__restrict__ cut_val, int Fpad,
                            size_t Npad, unsigned char *__restrict__ bins, unsigned char *__restrict__ binsT, int multi) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    for (int j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
        const int f = col[j];
        const float v = val[j];
        const int b0 = cut_ptr[f];
        int lo = b0, hi = cut_ptr[f + 1] - 1;
        if (hi < lo) continue;
        if (multi) lo = bin_search_down(cut_val, lo, hi, v);
        else
        while (lo < hi) {
            const int mid = lo + (hi - lo) / 2;
            if (cut_val[mid] <= v) lo = mid + 1; else hi = mid;
        }
        const unsigned char b = (unsigned char)(lo - b0);
        bins[(size_t)r * Fpad + f] = b;
        binsT[(size_t)f * Npad + r] = b;
    }
}

// Wide sparse data: the reference's own layout, one global bin id per stored value
// (hist_tree_builder_single.cu:113-119), sharing the CSR row pointers.
static __global__ void k_bin_csr(const int *__restrict__ col, const float *__restrict__ val, size_t nnz,
                                 const int *__restrict__ cut_ptr, const float *__restrict__ cut_val, int *__restrict__ out, int multi) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nnz; i += (size_t)gridDim.x * blockDim.x) {
        const int f = col[i];
        const float v = val[i];
        int lo = cut_ptr[f], hi = cut_ptr[f + 1] - 1;
        if (multi) lo = bin_search_down(cut_val, lo, hi, v);
        else
        while (lo < hi) {
            const int mid = lo + (hi - lo) / 2;
            if (cut_val[mid] <= v) lo = mid + 1; else hi = mid;
        }
        out[i] = lo;
    }
}

// flag = 1 when some row's bin ids do not ascend (the partition looks a feature up by binary search inside the row)
static __global__ void k_rows_unsorted(const int *__restrict__ row_ptr, const int *__restrict__ bin, int n_rows, int *__restrict__ flag) {
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
        bool bad = false;
        for (int i = row_ptr[r] + 1; i < row_ptr[r + 1]; ++i) bad |= bin[i - 1] > bin[i];
        if (bad) *flag = 1;
    }
}

// y[i] <- index of y[i] among the ascending `label` values, 0 when it is not one of them
// (DataSet::group_label, src/thundergbm/dataset.cpp:83-101)
static __global__ void k_map_labels(float *__restrict__ y, int n, const float *__restrict__ label, int n_label) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = y[i];
        int lo = 0, hi = n_label;
        while (lo < hi) {
            const int mid = (lo + hi) / 2;
            if (label[mid] < v) lo = mid + 1; else hi = mid;
        }
        y[i] = (lo < n_label && label[lo] == v) ? (float)lo : 0.f;
    }
}

// ------------------------------------------------------------------ objectives
// block-wide maximum of |g| and h, then one atomic pair per block (every thread of the block must call it)
__device__ inline void track_max(float ag, float h, unsigned *maxbits) {
    // non-negative floats order like their bit patterns
    __shared__ unsigned smax[2][32];
    unsigned a = __float_as_uint(ag), b = __float_as_uint(h);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a = max(a, __shfl_xor_sync(0xffffffffu, a, o));
        b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) { smax[0][warp] = a; smax[1][warp] = b; }
    __syncthreads();
    if (warp == 0) {
        a = lane < nw ? smax[0][lane] : 0u;
        b = lane < nw ? smax[1][lane] : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a = max(a, __shfl_xor_sync(0xffffffffu, a, o));
            b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
        }
        if (lane == 0) { atomicMax(maxbits, a); atomicMax(maxbits + 1, b); }
    }
}

// SquareLoss / LogisticLoss gradients (include/thundergbm/objective/regression_obj.h:129-154)
__device__ __forceinline__ float2 pointwise_gh(int logistic, float y, float yp) {
    if (logistic) {
        const float p = __fdiv_rn(1.0f, __fadd_rn(1.0f, portable_expf(-yp)));
        return make_float2(__fsub_rn(p, y), fmaxf(__fmul_rn(p, __fsub_rn(1.0f, p)), 1e-16f));
    }
    return make_float2(__fsub_rn(yp, y), 1.0f);
}

// one row's term of the training metric: squared error (pointwise_metric.cu:8-22), or 1 for a correct binary
// prediction (multiclass_metric.cu:9-46: sigmoid evaluated in double, class 1 above 0.5)
__device__ __forceinline__ double pointwise_metric_term(int objective, float y, float yp) {
    if (objective == BINARY_LOGISTIC) {
        // sigmoid(x) > 0.5 is decided by the sign of x except within rounding distance of zero
        const int k = fabsf(yp) > 1e-8f ? (yp > 0.f ? 1 : 0) : ((1.0 / (1.0 + exp(-(double)yp)) > 0.5) ? 1 : 0);
        return ((float)k == y) ? 1.0 : 0.0;
    }
    const float e = __fsub_rn(yp, y);
    return (double)__fmul_rn(e, e);
}

static __global__ void k_grad_pointwise(const float *__restrict__ y, const float *__restrict__ yp, int n, int logistic,
                                 float2 *__restrict__ gh, unsigned *__restrict__ maxbits) {
    float mg = 0.f, mh = 0.f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float2 v = pointwise_gh(logistic, y[i], yp[i]);
        const float g = v.x, h = v.y;
        gh[i] = make_float2(g, h);
        mg = fmaxf(mg, fabsf(g)); mh = fmaxf(mh, h);
    }
    track_max(mg, mh, maxbits);
}

// Softmax::get_gradient (src/thundergbm/objective/multiclass_obj.cu:7-35), class-major gh[k*N+i]
static __global__ void k_grad_softmax(const float *__restrict__ y, const float *__restrict__ yp, int n, int K,
                               float2 *__restrict__ gh, unsigned *__restrict__ maxbits) {
    float mg = 0.f, mh = 0.f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float mx = yp[i];
        for (int k = 1; k < K; ++k) mx = fmaxf(mx, yp[(size_t)k * n + i]);
        float sum = 0.f;
        for (int k = 0; k < K; ++k) sum = __fadd_rn(sum, portable_expf(__fsub_rn(yp[(size_t)k * n + i], mx)));
        const float yi = y[i];
        for (int k = 0; k < K; ++k) {
            const float p = __fdiv_rn(portable_expf(__fsub_rn(yp[(size_t)k * n + i], mx)), sum);
            const float g = ((float)k == yi) ? __fsub_rn(p, 1.0f) : p;
            const float h = fmaxf(__fmul_rn(__fmul_rn(2.0f, p), __fsub_rn(1.0f, p)), 1e-16f);
            gh[(size_t)k * n + i] = make_float2(g, h);
            mg = fmaxf(mg, fabsf(g));
            mh = fmaxf(mh, h);
        }
    }
    track_max(mg, mh, maxbits);
}

// Round the round's gradients to the fixed-point grid and sum them per class (root node sums,
// Tree::init2, src/thundergbm/tree.cu:31).  grid = (blocks, K)
//
// The rounding is dithered, q = floor(v * scale + u) with u in [0,1) a hash of (round, class, global row):
// round-to-nearest would move every row that carries the same gradient the same way (in the first round all rows
// of a class do), and those shifts would add up coherently in the histogram sums.
//
// `gh` null: the gradients are those of a pointwise objective (`logistic` 0/1) and are computed again from y and the
// scores here -- the pass that found their maxima (k_predict_walk) did not store them.
static __global__ void k_quantize(const float2 *__restrict__ gh, int n, const unsigned *__restrict__ maxbits, int quant_bits,
                           uint32_t round, uint32_t row_offset, int2 *__restrict__ ghq,
                           unsigned long long *__restrict__ root_sum, QuantInfo *__restrict__ qinfo,
                           const float *__restrict__ y, const float *__restrict__ yp, int logistic,
                           const RoundState *__restrict__ rs) {
    if (rs) round = (uint32_t)rs->round;  // the booster's rounds; the base-score pass gives its own
    const int k = blockIdx.y;
    const int eg = exp_above(__uint_as_float(maxbits[0])), eh = exp_above(__uint_as_float(maxbits[1]));
    const double sg = pow2d(quant_bits - eg), sh = pow2d(quant_bits - eh);
    if (blockIdx.x == 0 && k == 0 && threadIdx.x == 0) {
        qinfo->sg = sg; qinfo->sh = sh;
        qinfo->inv_sg = pow2d(eg - quant_bits); qinfo->inv_sh = pow2d(eh - quant_bits);
    }
    long long tg = 0, th = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float2 v = gh ? gh[(size_t)k * n + i] : pointwise_gh(logistic, y[i], yp[i]);
        const uint32_t row = row_offset + (uint32_t)i;
        const double ug = (double)mix32(0x9E3779B9u, round, (uint32_t)k, row) * (1.0 / 4294967296.0);
        const double uh = (double)mix32(0x9E3779B9u + 1u, round, (uint32_t)k, row) * (1.0 / 4294967296.0);
        const int qg = (int)__double2ll_rd((double)v.x * sg + ug), qh = (int)__double2ll_rd((double)v.y * sh + uh);
        ghq[(size_t)k * n + i] = make_int2(qg, qh);
        tg += qg; th += qh;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { tg += shfl_xor_ll(tg, o); th += shfl_xor_ll(th, o); }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(root_sum + 2 * k, (unsigned long long)tg);
        atomicAdd(root_sum + 2 * k + 1, (unsigned long long)th);
    }
}


// ------------------------------------------------------------------ row and column sampling
// RowSampler::do_bagging (src/thundergbm/row_sampler.cu:9-35): M = size of the gradient array (num_class x rows) draws
// of a uniform index into that array, every entry's (g,h) multiplied by the number of times it was drawn.  The
// reference seeds thrust's generator from std::rand(); here draw j of round r is a counter-based hash, so that the
// CPU restatement and any number of ranks draw the same sample.  Every rank makes all the draws and keeps those that
// land in its own rows.  entry = class * n_global + global row.
static __global__ void k_bag_draw(unsigned long long m_total, uint32_t seed, const RoundState *__restrict__ rs, long long n_global,
                                  long long row_offset, int n_local, int K, int *__restrict__ count) {
    const uint32_t round = (uint32_t)rs->round;
    for (unsigned long long j = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; j < m_total; j += (unsigned long long)gridDim.x * blockDim.x) {
        const uint32_t r = mix32(seed ^ 0xBA661D6Eu, round, (uint32_t)(j >> 32), (uint32_t)j);
        const unsigned long long e = ((unsigned long long)r * m_total) >> 32;
        const long long k = (long long)(e / (unsigned long long)n_global), row = (long long)(e % (unsigned long long)n_global) - row_offset;
        if (k < K && row >= 0 && row < n_local) atomicAdd(count + k * n_local + row, 1);
    }
}
// gh *= multiplicity; also the maxima of the scaled gradients for the fixed-point grid (every thread of the block calls track_max)
static __global__ void k_bag_scale(float2 *__restrict__ gh, const int *__restrict__ count, size_t n, unsigned *__restrict__ maxbits) {
    float mg = 0.f, mh = 0.f;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float2 v = gh[i];
        const float c = (float)count[i];
        v.x = __fmul_rn(v.x, c); v.y = __fmul_rn(v.y, c);
        gh[i] = v;
        mg = fmaxf(mg, fabsf(v.x)); mh = fmaxf(mh, v.y);
    }
    track_max(mg, mh, maxbits);
}

// ------------------------------------------------------------------ tree set-up
// Tree::init2 (src/thundergbm/tree.cu:8-39)
// root_is_f64: fp32 mode, the root sums are doubles (k_sum_gh_final) instead of integers on the fixed-point grid
static __global__ void k_tree_init(TreeNode *__restrict__ nodes, int n_nodes, const unsigned long long *__restrict__ root_sum,
                            const QuantInfo *__restrict__ q, float lambda, int n_rows, int *__restrict__ seg_begin,
                            int *__restrict__ seg_cnt, int *__restrict__ gcnt, TreeCtl *__restrict__ ctl, int root_is_f64) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_nodes) return;
    TreeNode t;
    memset(&t, 0, sizeof(t));
    t.final_id = i;
    t.split_feature_id = -1;
    t.parent_index = i == 0 ? -1 : (i - 1) / 2;
    if (i < n_nodes / 2) { t.is_leaf = 0; t.lch_index = 2 * i + 1; t.rch_index = 2 * i + 2; }
    else { t.is_leaf = 1; t.lch_index = -1; t.rch_index = -1; }
    if (i == 0) {
        if (root_is_f64) {
            t.sum_g = __double2float_rn(__longlong_as_double((long long)root_sum[0]));
            t.sum_h = __double2float_rn(__longlong_as_double((long long)root_sum[1]));
        } else {
            t.sum_g = q2f((long long)root_sum[0], q->inv_sg);
            t.sum_h = q2f((long long)root_sum[1], q->inv_sh);
        }
        t.is_valid = 1;
        t.base_weight = __fdiv_rn(-t.sum_g, __fadd_rn(t.sum_h, lambda));
        seg_begin[0] = 0; seg_cnt[0] = n_rows; gcnt[0] = n_rows;
        ctl->n_records = n_rows;
    }
    nodes[i] = t;
}

// ------------------------------------------------------------------ histogram build
// Exclusive prefix sums over n values inside one block of 1024 threads: out(i, prefix before i); returns the total.
// `scratch` holds 33 ints of shared memory.  Every thread of the block must call it.
template <typename In, typename Out>
__device__ inline int block_scan_excl(int n, In in, Out out, int *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int carry = 0;
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        const int x = i < n ? in(i) : 0;
        int v = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
        __syncthreads();
        if (lane == 31) scratch[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int t = scratch[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, t, o); if (lane >= o) t += u; }
            scratch[lane] = t;
        }
        __syncthreads();
        const int incl = v + (warp ? scratch[warp - 1] : 0) + carry;
        if (i < n) out(i, incl - x);
        carry += scratch[31];
    }
    __syncthreads();
    return carry;
}

// Order in which the dense histogram kernel visits the level's tiles.
// The tiles are dealt out to `n_ctas * HIST_SHARES` shares in proportion to the items' sizes (cumulative rounding, so
// the shares of different items are disjoint; an item too small for a share of its own rides on one).  Inside an item
// tile t belongs to share v0 + t mod k.  CTA c owns HIST_SHARES consecutive shares and visits, item by item, the tiles
// of its shares in ascending order: every CTA walks each of its (one or two, rarely more) lists once, front to back,
// and since all CTAs carry about the same number of tiles, all lists are walked at the same relative pace.  Row ids
// ascend inside every list, so at any time the whole GPU gathers rows from one moving window of the bin matrix:
// DRAM pages and 64-byte sectors get shared between nodes.  A pure gather of 5.2 M of 10.5 M rows in 8 to 64 lists
// takes 72 us this way and 100 to 110 us list after list.
// Output: seq[cta_off[c] .. cta_off[c+1]) = the tiles of CTA c as (first record, records, slab, 0).
// tile_base[0..nw] must be complete.  Called by every thread of a 1024-thread block.
__device__ inline void hist_sequence(int nw, int tiles, HistWork *__restrict__ work, const int *__restrict__ tile_base,
                                     int n_ctas, int *__restrict__ cta_off, int4 *__restrict__ seq, int *scratch) {
    const int n_shares = n_ctas * HIST_SHARES;
    for (int w = threadIdx.x; w < nw; w += 1024) {
        const long long t0 = tile_base[w], t1 = tile_base[w + 1];
        int v0 = tiles ? (int)((t0 * n_shares + tiles / 2) / tiles) : 0;
        const int v1 = tiles ? (int)((t1 * n_shares + tiles / 2) / tiles) : 0;
        int k = v1 - v0;
        if (k <= 0) { k = 1; v0 = min(v0, n_shares - 1); }
        work[w].vk = v0 | (k << 16);
    }
    __syncthreads();
    // items with a share among the CTA's: first item whose last share is >= va ... first item whose first share is >= vb
    auto items_of = [&](int c, int &ib, int &ie) {
        const int va = c * HIST_SHARES, vb = va + HIST_SHARES;
        int lo = 0, hi = nw;
        while (lo < hi) {
            const int mid = (lo + hi) / 2, vk = work[mid].vk;
            if ((vk & 0xffff) + (vk >> 16) - 1 >= va) hi = mid; else lo = mid + 1;
        }
        ib = lo;
        hi = nw;
        while (lo < hi) {
            const int mid = (lo + hi) / 2;
            if ((work[mid].vk & 0xffff) >= vb) hi = mid; else lo = mid + 1;
        }
        ie = lo;
    };
    // the CTA's part of item w: residues [ra, ra + width) mod k, `count` tiles
    auto part_of = [&](int c, int w, int &k, int &ra, int &width) {
        const int va = c * HIST_SHARES, vb = va + HIST_SHARES;
        const int vk = work[w].vk, v0 = vk & 0xffff, T = tile_base[w + 1] - tile_base[w];
        k = vk >> 16;
        ra = max(va, v0) - v0;
        width = min(vb, v0 + k) - v0 - ra;
        return (T / k) * width + min(max(T % k - ra, 0), width);
    };
    __shared__ int sh_ib[HIST_MAX_CTAS], sh_ie[HIST_MAX_CTAS];  // the searches are chains of dependent loads: done once
    block_scan_excl(n_ctas,
                    [&](int c) {
                        int ib, ie, n = 0, k, ra, width;
                        items_of(c, ib, ie);
                        sh_ib[c] = ib; sh_ie[c] = ie;
                        for (int w = ib; w < ie; ++w) n += part_of(c, w, k, ra, width);
                        return n;
                    },
                    [&](int c, int excl) { cta_off[c] = excl; }, scratch);
    if (threadIdx.x == 0) cta_off[n_ctas] = tiles;
    __syncthreads();
    // one warp writes the sequence of one CTA, 32 tiles at a time
    const int lane = threadIdx.x & 31;
    for (int c = threadIdx.x >> 5; c < n_ctas; c += 32) {
        const int ib = sh_ib[c], ie = sh_ie[c];
        int pos = cta_off[c];
        for (int w = ib; w < ie; ++w) {
            int k, ra, width;
            const int count = part_of(c, w, k, ra, width);
            const HistWork it = work[w];
            for (int n = lane; n < count; n += 32) {
                const int t = (n / width) * k + ra + n % width;
                seq[pos + n] = make_int4(it.begin + t * HIST_THREADS, min(HIST_THREADS, it.count - t * HIST_THREADS), it.slab, 0);
            }
            pos += count;
        }
    }
}

// Which sibling to build (the one with fewer rows over all ranks, ties -> left:
// hist_tree_builder_single.cu:466) and the work list of the level.  Called by every thread of a 1024-thread block.
__device__ inline void hist_plan(int level, const int *__restrict__ seg_begin, const int *__restrict__ seg_cnt,
                                 const int *__restrict__ gcnt, const TreeNode *__restrict__ nodes, int by_hessian,
                                 int *__restrict__ built_right, HistWork *__restrict__ work, int *__restrict__ tile_base,
                                 TreeCtl *__restrict__ ctl, int n_ctas, int *__restrict__ cta_off, int4 *__restrict__ seq) {
    __shared__ int scratch[33];
    __shared__ unsigned long long rows;
    if (level == 0) {
        const int tiles0 = (seg_cnt[0] + HIST_THREADS - 1) / HIST_THREADS;
        if (threadIdx.x == 0) {
            work[0] = HistWork{0, seg_cnt[0], 0, 0};
            tile_base[0] = 0;
            tile_base[1] = tiles0;
            built_right[0] = 0;
            ctl->stat_rows_root += seg_cnt[0];
            ctl->stat_hists += 1;
            ctl->n_hist_work = 1;
            ctl->n_hist_tiles = tiles0;
        }
        __syncthreads();
        hist_sequence(1, tiles0, work, tile_base, n_ctas, cta_off, seq, scratch);
        return;
    }
    const int pairs = 1 << (level - 1);
    if (threadIdx.x == 0) rows = 0;
    __syncthreads();
    // -1: nothing to do, else which child is built.  One rank: the child with fewer rows, like the reference.
    // Several ranks: the row counts are rank-local, so every rank takes the child with the smaller hessian sum from
    // the replicated node table -- the same choice everywhere without a collective.  All histogram sums are exact
    // integers, so built and subtracted histograms are identical whichever sibling is built.
    auto right_of = [&](int j) {
        if (by_hessian) {
            const int off = (1 << level) - 1;
            const TreeNode &l = nodes[off + 2 * j], &r = nodes[off + 2 * j + 1];
            if (!l.is_valid || !r.is_valid) return -1;
            return l.sum_h > r.sum_h ? 1 : 0;
        }
        const int gl = gcnt[2 * j], gr = gcnt[2 * j + 1];
        return max(gl, gr) == 0 ? -1 : (gl > gr ? 1 : 0);
    };
    // compacted position of every active pair in the work list
    const int nw = block_scan_excl(pairs, [&](int j) { return right_of(j) >= 0 ? 1 : 0; },
                                   [&](int j, int pos) {
                                       const int r = right_of(j);
                                       built_right[j] = r;
                                       if (r >= 0) {
                                           const int c = 2 * j + r;
                                           work[pos] = HistWork{seg_begin[c], seg_cnt[c], j, 0};
                                           atomicAdd(&rows, (unsigned long long)seg_cnt[c]);
                                       }
                                   }, scratch);
    const int tiles = block_scan_excl(nw, [&](int w) { return (work[w].count + HIST_THREADS - 1) / HIST_THREADS; },
                                      [&](int w, int base) { tile_base[w] = base; }, scratch);
    if (threadIdx.x == 0) {
        tile_base[nw] = tiles;
        ctl->stat_rows_gather += rows;
        ctl->stat_hists += nw;
        ctl->n_hist_work = nw;
        ctl->n_hist_tiles = tiles;
    }
    __syncthreads();
    hist_sequence(nw, tiles, work, tile_base, n_ctas, cta_off, seq, scratch);
}

// Permute the 16 bin bytes of a half row so that byte j of the register array is the bin of slot (j XOR key),
// key = 0..15: at step j the 16 lane pairs of a warp then address 16 different slots of either half.  Key bits 0-1
// permute the bytes inside every word (one PRMT each), bits 2-3 exchange whole words.
__device__ __forceinline__ void xor_permute_half(uint32_t (&w)[4], int key) {
    const uint32_t sel = (key & 2) ? ((key & 1) ? 0x0123u : 0x1032u) : ((key & 1) ? 0x2301u : 0x3210u);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __byte_perm(w[i], 0u, sel);
    const int hi = key >> 2;
#pragma unroll
    for (int s = 1; s <= 2; s <<= 1) {
        uint32_t t[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) t[i] = (hi & s) ? w[i ^ s] : w[i];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = t[i];
    }
}

// Histogram build of one level (root: hist_tree_builder_single.cu:203-216, deeper levels: :485-505).
// Persistent CTAs, one per SM; grid = (ctas, feature groups of 32).  Each CTA visits the tiles the level's plan
// gave it (see hist_sequence).  A lane holds one 16-feature half of two rows; the shared-memory
// accumulators are laid out [bin][32 features] so that the bank is the feature index, and at step j the 32 lanes
// of a warp handle 32 different features, so every shared atomic of a warp hits 32 different banks.  Accumulators are int32.  Before they could overflow
// (`window_rows` rows of at most 2^quant_bits each) they are drained into int64 totals, also in shared
// memory; the totals go to the node's int64 histogram in global memory when the CTA moves on to another
// node and at the end.
template <bool GATHER>
static __global__ void __launch_bounds__(HIST_THREADS, 1)
k_hist(const unsigned char *__restrict__ bins, int Fpad, int F, const int *__restrict__ rec_idx,
       const int2 *__restrict__ rec_gh, const int *__restrict__ cta_off, const int4 *__restrict__ seq,
       const int *__restrict__ cut_ptr, const int *__restrict__ cut_fid,
       long long *__restrict__ slab, int B, int window_rows) {
    extern __shared__ __align__(16) int sh_hist[];  // int32 g,h: [2][256][32]; int64 totals g,h: [2][256][32]
    int *acc = sh_hist;
    int *hg = acc;  // g accumulators; the h accumulators follow at +256*32
    long long *tot = reinterpret_cast<long long *>(sh_hist + 2 * 256 * 32);

    const int group = blockIdx.y;
    const int f0 = group * 32;
    const int nf = min(32, F - f0);
    const int lane = threadIdx.x & 31;
    const int i2 = cta_off[blockIdx.x], i_end = cta_off[blockIdx.x + 1];  // the CTA's tiles in seq[], see hist_sequence
    if (i2 >= i_end) return;
    for (int i = threadIdx.x; i < 2 * 256 * 32; i += HIST_THREADS) { acc[i] = 0; tot[i] = 0; }
    __syncthreads();

    auto drain = [&]() {  // int32 window -> int64 totals, same [bin][feature] layout
        __syncthreads();
#pragma unroll 4
        for (int i = threadIdx.x; i < 2 * 256 * 32; i += HIST_THREADS) {
            const int v = acc[i];
            if (v) { tot[i] += v; acc[i] = 0; }
        }
        __syncthreads();
    };
    // totals + open window -> the node's histogram.  A thread keeps one feature (its bank) and walks the local bins,
    // so the loop has no dependent loads; everything it reads is zeroed for the next node.
    const int flush_f = threadIdx.x & 31;
    const int flush_b0 = flush_f < nf ? cut_ptr[f0 + flush_f] : 0;
    const int flush_nb = flush_f < nf ? cut_ptr[f0 + flush_f + 1] - flush_b0 : 0;
    auto flush = [&](int slab_idx) {
        __syncthreads();
        unsigned long long *dst = reinterpret_cast<unsigned long long *>(slab + ((size_t)slab_idx * B + flush_b0) * 2);
#pragma unroll 2
        for (int i = threadIdx.x >> 5; i < 256; i += HIST_THREADS / 32) {
            const int s = i * 32 + flush_f;
            const long long vg = tot[s] + acc[s], vh = tot[256 * 32 + s] + acc[256 * 32 + s];
            tot[s] = 0; tot[256 * 32 + s] = 0; acc[s] = 0; acc[256 * 32 + s] = 0;
            if (i < flush_nb) {
                if (vg) atomicAdd(dst + 2 * i, (unsigned long long)vg);
                if (vh) atomicAdd(dst + 2 * i + 1, (unsigned long long)vh);
            }
        }
        __syncthreads();
    };

    // Two lanes share a row: lane l loads the 16-byte half (l & 1) of the rows at tile positions
    // warp*32 + (l >> 1) ("A") and 16 further on ("B").  One load instruction of a warp therefore touches 16 rows
    // (16 sectors) instead of 32 half-used ones, which halves the L1 wavefronts the gathered rows cost.
    const int qa = (threadIdx.x & ~31) | (lane >> 1), qb = qa + 16;  // the lane's two tile positions
    const uint32_t laneoff = ((uint32_t)(lane & 1) << 6) | ((uint32_t)(lane >> 1) << 2);  // 4 * (16*half + key)
    // Software pipeline over the CTA's tiles.  While tile i is accumulated, the bin rows of tile i+1 are on their
    // way into registers, those of tile i+2 have been asked into L2 (a prefetch holds no register), and the row ids
    // of tile i+3 are being fetched.  The gather levels are bound by the bytes in flight (a loaded DRAM access takes
    // 2-3 us here): one tile per warp in registers alone sustains only ~2.4 TB/s of sector traffic.
    // ids(): row ids of the lane's two positions in tile i, -1 = no record
    auto ids = [&](int i, int &ra, int &rb) {
        ra = rb = -1;
        if (i < i_end) {
            const int4 e = seq[i];
            if (qa < e.y) ra = GATHER ? rec_idx[e.x + qa] : e.x + qa;
            if (qb < e.y) rb = GATHER ? rec_idx[e.x + qb] : e.x + qb;
        }
    };
    const size_t half_off = (size_t)f0 + 16u * (lane & 1);
    uint4 na = make_uint4(0, 0, 0, 0), nb = na;
    int2 nva = make_int2(0, 0), nvb = nva;
    bool noka = false, nokb = false;
    int slab1 = 0;
    int r1a, r1b, r2a, r2b;
    auto load_rows = [&](int i) {  // rows of tile i (ids r1a, r1b) -> registers
        noka = r1a >= 0; nokb = r1b >= 0;
        if (i < i_end) {
            const int4 e = seq[i];
            slab1 = e.z;
            if (noka) { na = *reinterpret_cast<const uint4 *>(bins + (size_t)r1a * Fpad + half_off); nva = rec_gh[e.x + qa]; }
            if (nokb) { nb = *reinterpret_cast<const uint4 *>(bins + (size_t)r1b * Fpad + half_off); nvb = rec_gh[e.x + qb]; }
        }
    };
    auto prefetch_rows = [&]() {  // rows with ids r2a, r2b -> L2; one lane of each pair asks for the row's sector
        if (GATHER && !(lane & 1)) {
            if (r2a >= 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(bins + (size_t)r2a * Fpad + f0));
            if (r2b >= 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(bins + (size_t)r2b * Fpad + f0));
        }
    };
    int i = i2;
    ids(i, r1a, r1b);
    ids(i + 1, r2a, r2b);
    load_rows(i);
    prefetch_rows();
    r1a = r2a; r1b = r2b;
    ids(i + 2, r2a, r2b);
    int slab_cur = slab1;
    int since = 0;
    for (; i < i_end; ++i) {
        const uint4 a = na, b = nb;
        const int2 va = nva, vb = nvb;
        const bool oka = noka, okb = nokb;
        const int slab_this = slab1;
        load_rows(i + 1);
        prefetch_rows();
        r1a = r2a; r1b = r2b;
        ids(i + 3, r2a, r2b);
        if (slab_this != slab_cur) {  // the tile belongs to another node: hand the finished one over
            flush(slab_cur);
            slab_cur = slab_this;
            since = 0;
        } else if (since + HIST_THREADS > window_rows) {
            drain();
            since = 0;
        }
        since += HIST_THREADS;
        // Step j adds a row to (bin of feature 16*half + (j ^ key), that feature), key = lane >> 1: the 32 lanes of a
        // warp address 32 different features = 32 different banks.  Byte offset of the accumulator:
        // bin * 128 | feature * 4 -- the bin field comes straight out of the packed word with one shift and one
        // mask.  No test for missing values: bin 255 (missing, and the padding columns beyond F) lands in row 255
        // of the table, which no feature ever reads back.
        char *const gbase = reinterpret_cast<char *>(hg);
        if (oka) {
            uint32_t w[4] = {a.x, a.y, a.z, a.w};
            xor_permute_half(w, lane >> 1);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t word = w[j >> 2];
                const uint32_t binoff = ((j & 3) == 0 ? (word << 7) : (word >> (8 * (j & 3) - 7))) & 0x7f80u;
                const uint32_t off = binoff | (laneoff ^ (4u * j));
                atomicAdd(reinterpret_cast<int *>(gbase + off), va.x);
                atomicAdd(reinterpret_cast<int *>(gbase + off + 256 * 32 * 4), va.y);
            }
        }
        if (okb) {
            uint32_t w[4] = {b.x, b.y, b.z, b.w};
            xor_permute_half(w, lane >> 1);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t word = w[j >> 2];
                const uint32_t binoff = ((j & 3) == 0 ? (word << 7) : (word >> (8 * (j & 3) - 7))) & 0x7f80u;
                const uint32_t off = binoff | (laneoff ^ (4u * j));
                atomicAdd(reinterpret_cast<int *>(gbase + off), vb.x);
                atomicAdd(reinterpret_cast<int *>(gbase + off + 256 * 32 * 4), vb.y);
            }
        }
    }
    flush(slab_cur);
}

// Histogram build for the wide sparse layout (CSR of global bin ids).  A histogram of ~100k bins does not fit in
// shared memory; with Zipf-like column frequencies most updates hit the lowest column ids, so the first
// SPARSE_SMEM_BINS bins are accumulated per CTA in shared memory (int64 atomics) and the long tail goes straight to
// the node's histogram with global int64 atomics (L2-resident: 16 B per bin).  One warp per row, lanes over its values.
constexpr int SPARSE_SMEM_BINS = 12288;  // 192 KB of int64 (g, h) cells
constexpr int SPARSE_THREADS = 1024;    // one CTA per SM

template <bool GATHER>
static __global__ void __launch_bounds__(SPARSE_THREADS, 1)
k_hist_sparse(const int *__restrict__ row_ptr, const int *__restrict__ bin, const int *__restrict__ rec_idx,
              const int2 *__restrict__ rec_gh, const HistWork *__restrict__ work, const int *__restrict__ tile_base,
              const TreeCtl *__restrict__ ctl, long long *__restrict__ slab, int B) {
    extern __shared__ __align__(16) long long sh_sparse[];  // [SPARSE_SMEM_BINS][2]
    const int nsm = min(B, SPARSE_SMEM_BINS);
    const int total = ctl->n_hist_tiles, nwork = ctl->n_hist_work;
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int t_begin = min(total, (int)blockIdx.x * per), t_end = min(total, t_begin + per);
    if (t_begin >= t_end) return;
    for (int i = threadIdx.x; i < 2 * nsm; i += SPARSE_THREADS) sh_sparse[i] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto flush = [&](int slab_idx) {
        __syncthreads();
        long long *dst = slab + (size_t)slab_idx * B * 2;
        for (int i = threadIdx.x; i < 2 * nsm; i += SPARSE_THREADS) {
            const long long v = sh_sparse[i];
            if (v) { atomicAdd(reinterpret_cast<unsigned long long *>(dst + i), (unsigned long long)v); sh_sparse[i] = 0; }
        }
        __syncthreads();
    };
    int w = 0;
    {
        int lo = 0, hi = nwork - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) / 2;
            if (tile_base[mid] <= t_begin) lo = mid; else hi = mid - 1;
        }
        w = lo;
    }
    int w_cur = w;
    for (int t = t_begin; t < t_end; ++t) {
        while (w + 1 < nwork && t >= tile_base[w + 1]) ++w;
        if (w != w_cur) { flush(work[w_cur].slab); w_cur = w; }
        const HistWork it = work[w];
        long long *dst = slab + (size_t)it.slab * B * 2;
        const int first = (t - tile_base[w]) * HIST_THREADS;
        const int last = min(it.count, first + HIST_THREADS);
        // A warp takes every 32nd row of the tile.  Three rows are in flight per warp: the row pointers and gradients
        // of the row after next, the first 32 bin ids of the next row, and the row being accumulated -- a row is a
        // chain of three dependent loads (record -> row pointers -> bin ids) and would otherwise cost three memory
        // latencies each.
        constexpr int W = SPARSE_THREADS / 32;
        auto meta = [&](int q, int &j0, int &j1, int2 &v) {
            j0 = j1 = 0; v = make_int2(0, 0);
            if (q < last) {
                const int p = it.begin + q;
                const int r = GATHER ? rec_idx[p] : p;
                v = rec_gh[p];
                j0 = row_ptr[r]; j1 = row_ptr[r + 1];
            }
        };
        int q = first + warp;
        int j0, j1, nj0, nj1, mj0, mj1;
        int2 v, nv, mv;
        meta(q, j0, j1, v);
        meta(q + W, nj0, nj1, nv);
        int b0 = j0 + lane < j1 ? bin[j0 + lane] : -1;
        for (; q < last; q += W) {
            meta(q + 2 * W, mj0, mj1, mv);
            const int nb0 = nj0 + lane < nj1 ? bin[nj0 + lane] : -1;
            int b = b0;
            for (int j = j0 + lane; j < j1; j += 32) {
                if (j != j0 + lane) b = bin[j];
                if (b < nsm) {
                    atomicAdd(reinterpret_cast<unsigned long long *>(sh_sparse + 2 * b), (unsigned long long)(long long)v.x);
                    atomicAdd(reinterpret_cast<unsigned long long *>(sh_sparse + 2 * b + 1), (unsigned long long)(long long)v.y);
                } else {
                    atomicAdd(reinterpret_cast<unsigned long long *>(dst + 2 * b), (unsigned long long)(long long)v.x);
                    atomicAdd(reinterpret_cast<unsigned long long *>(dst + 2 * b + 1), (unsigned long long)(long long)v.y);
                }
            }
            j0 = nj0; j1 = nj1; v = nv; b0 = nb0;
            nj0 = mj0; nj1 = mj1; nv = mv;
        }
    }
    flush(work[w_cur].slab);
}

// ------------------------------------------------------------------ split evaluation
// Histogram cells are `long long` sums on the round's fixed-point grid (exact mode) or `float` sums (fp32 mode, the
// reference's own arithmetic: GHPair of floats, include/thundergbm/common.h:43-59).  The evaluation kernels are
// written once over the cell type.
template <typename T> __device__ __forceinline__ double cell_inv(const QuantInfo *q, int h);
template <> __device__ __forceinline__ double cell_inv<long long>(const QuantInfo *q, int h) { return h ? q->inv_sh : q->inv_sg; }
template <> __device__ __forceinline__ double cell_inv<float>(const QuantInfo *, int) { return 1.0; }
__device__ __forceinline__ float cell_f(long long v, double inv_scale) { return q2f(v, inv_scale); }
__device__ __forceinline__ float cell_f(float v, double) { return v; }
__device__ __forceinline__ long long shfl_up_t(long long v, int d) { return shfl_up_ll(v, d); }
__device__ __forceinline__ float shfl_up_t(float v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ __forceinline__ long long shfl_t(long long v, int src) { return shfl_ll(v, src); }
__device__ __forceinline__ float shfl_t(float v, int src) { return __shfl_sync(0xffffffffu, v, src); }

__device__ __forceinline__ float split_gain(float pg, float ph, float lg, float lh, float rg, float rh, float mcw, float lam) {
    // compute_gain, hist_tree_builder_single.cu:279-286 (no fused multiply-add: products feed divisions)
    if (lh >= mcw && rh >= mcw)
        return __fsub_rn(__fadd_rn(__fdiv_rn(__fmul_rn(lg, lg), __fadd_rn(lh, lam)), __fdiv_rn(__fmul_rn(rg, rg), __fadd_rn(rh, lam))),
                         __fdiv_rn(__fmul_rn(pg, pg), __fadd_rn(ph, lam)));
    return 0.f;
}

// Sibling subtraction, per-feature prefix scan, missing sums, gains and per-feature argmax
// (hist_tree_builder_single.cu:257-347 for the root, :538-540 and :614-704 for sibling pairs).
// grid = (F, pairs); block = 64: warp 0 evaluates the left child, warp 1 the right child.
template <typename T>
__device__ __forceinline__ void eval_feature(int level, int F, int B, const int *__restrict__ cut_ptr, const TreeNode *nodes,
                                             const int *__restrict__ built_right, const T *__restrict__ built,
                                             const T *__restrict__ parent, T *__restrict__ full,
                                             const QuantInfo *__restrict__ q, float mcw, float lam, SplitRec *recs, int bs,
                                             const unsigned char *__restrict__ ignored, int multi) {
    // multi: the column-sharded builder's candidates (hist_tree_builder.cu:299-352): the INCLUSIVE prefix along the
    // bins (they count down from the largest values there) is the right child, the left one is the node minus it,
    // missing values join the right child when that gains at least as much; the record then carries the right sums
    // bs: distance of two cells of `built` in cells (1 unless the fp32 histogram kernel spread them out)
    // ignored: the round's column-sampling mask (Shard::column_sampling, src/thundergbm/builder/shard.cu:8-23; the
    // masked features take no part in the split search, hist_tree_builder_single.cu:304,663), or null
    __shared__ T sg[2][256], sh[2][256];
    const int f = blockIdx.x, j = blockIdx.y;
    const int b0 = cut_ptr[f], nb = cut_ptr[f + 1] - b0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_children = level == 0 ? 1 : 2;
    const int node_local = level == 0 ? 0 : 2 * j + warp;
    const int off = (1 << level) - 1;
    SplitRec none = {0.f, -1, 0.f, 0.f, 0.f, 0.f};
    const int br = built_right[j];
    if (nb == 0 || br < 0 || (ignored && ignored[f])) {
        if (lane == 0 && warp < n_children) recs[(size_t)node_local * F + f] = none;
        return;
    }
    // asked for now, used after the histogram loads below: one memory latency instead of two
    const TreeNode nd = nodes[off + (warp < n_children ? node_local : 0)];
    const double inv_sg = cell_inv<T>(q, 0), inv_sh = cell_inv<T>(q, 1);
    if (level == 0) {
        for (int i = threadIdx.x; i < nb; i += 64) {
            const T cg = built[(size_t)2 * bs * (b0 + i)], ch = built[(size_t)2 * bs * (b0 + i) + 1];
            sg[0][i] = cg; sh[0][i] = ch;
            if (bs != 1) { full[2 * (b0 + i)] = cg; full[2 * (b0 + i) + 1] = ch; }  // the compact copy the next level subtracts from
        }
    } else {
        const T *bp = built + (size_t)j * B * 2 * bs, *pp = parent + (size_t)j * B * 2;
        T *fb = full + (size_t)(2 * j + br) * B * 2, *fo = full + (size_t)(2 * j + 1 - br) * B * 2;
        for (int i = threadIdx.x; i < nb; i += 64) {
            const T cg = bp[(size_t)2 * bs * (b0 + i)], ch = bp[(size_t)2 * bs * (b0 + i) + 1];
            const T og = pp[2 * (b0 + i)] - cg, oh = pp[2 * (b0 + i) + 1] - ch;
            sg[br][i] = cg; sh[br][i] = ch;
            sg[1 - br][i] = og; sh[1 - br][i] = oh;
            fb[2 * (b0 + i)] = cg; fb[2 * (b0 + i) + 1] = ch;
            fo[2 * (b0 + i)] = og; fo[2 * (b0 + i) + 1] = oh;
        }
    }
    __syncthreads();
    if (warp >= n_children) return;
    if (!nd.is_valid) {
        if (lane == 0) recs[(size_t)node_local * F + f] = none;
        return;
    }
    // each lane owns 8 consecutive bins
    T lg8[8], lh8[8];
    T tg = 0, th = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int b = lane * 8 + i;
        lg8[i] = tg; lh8[i] = th;  // exclusive prefix inside the lane
        if (b < nb) { tg += sg[warp][b]; th += sh[warp][b]; }
    }
    T ig = tg, ih = th;  // inclusive scan of the lane totals
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T ug = shfl_up_t(ig, o), uh = shfl_up_t(ih, o);
        if (lane >= o) { ig += ug; ih += uh; }
    }
    // prefix before the lane's first bin = inclusive value of the lane before (float cells: no subtraction of the
    // lane's own total, which would round)
    T base_g = shfl_up_t(ig, 1), base_h = shfl_up_t(ih, 1);
    if (lane == 0) { base_g = 0; base_h = 0; }
    const T tot_g = shfl_t(ig, 31), tot_h = shfl_t(ih, 31);
    const float pg = nd.sum_g, ph = nd.sum_h;
    const float mg = __fsub_rn(pg, cell_f(tot_g, inv_sg)), mh = __fsub_rn(ph, cell_f(tot_h, inv_sh));
    float best = 0.f, best_lg = 0.f, best_lh = 0.f;
    int best_bin = -1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int b = lane * 8 + i;
        if (b < nb && multi) {
            const float rg = cell_f(base_g + lg8[i] + sg[warp][b], inv_sg), rh = cell_f(base_h + lh8[i] + sh[warp][b], inv_sh);
            const float gl = fmaxf(0.f, split_gain(pg, ph, __fsub_rn(pg, rg), __fsub_rn(ph, rh), rg, rh, mcw, lam));
            const float rg2 = __fadd_rn(rg, mg), rh2 = __fadd_rn(rh, mh);
            const float gr = fmaxf(0.f, split_gain(pg, ph, __fsub_rn(pg, rg2), __fsub_rn(ph, rh2), rg2, rh2, mcw, lam));
            const float gn = gl > gr ? gl : -gr;
            if (best_bin < 0 || fabsf(gn) > fabsf(best)) { best = gn; best_bin = b; best_lg = rg; best_lh = rh; }
        } else if (b < nb) {
            const float lg = cell_f(base_g + lg8[i], inv_sg), lh = cell_f(base_h + lh8[i], inv_sh);
            const float gr = fmaxf(0.f, split_gain(pg, ph, lg, lh, __fsub_rn(pg, lg), __fsub_rn(ph, lh), mcw, lam));
            const float lg2 = __fadd_rn(lg, mg), lh2 = __fadd_rn(lh, mh);
            const float gl = fmaxf(0.f, split_gain(pg, ph, lg2, lh2, __fsub_rn(pg, lg2), __fsub_rn(ph, lh2), mcw, lam));
            const float gn = gl > gr ? gl : -gr;
            if (best_bin < 0 || fabsf(gn) > fabsf(best)) { best = gn; best_bin = b; best_lg = lg; best_lh = lh; }
        }
    }
    // warp arg-abs-max, ties -> smaller bin (hist_tree_builder_single.cu:330-335)
    unsigned long long key = best_bin < 0 ? 0ull
                                          : (((unsigned long long)__float_as_uint(fabsf(best)) << 32) | (unsigned)(0x7fffffff - best_bin));
    unsigned long long mk = key;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = (unsigned long long)shfl_xor_ll((long long)mk, o);
        mk = other > mk ? other : mk;
    }
    const unsigned win = __ballot_sync(0xffffffffu, key == mk && best_bin >= 0);
    const int src = __ffs(win) - 1;
    best = __shfl_sync(0xffffffffu, best, src);
    best_bin = __shfl_sync(0xffffffffu, best_bin, src);
    best_lg = __shfl_sync(0xffffffffu, best_lg, src);
    best_lh = __shfl_sync(0xffffffffu, best_lh, src);
    if (lane == 0) recs[(size_t)node_local * F + f] = SplitRec{best, best_bin, best_lg, best_lh, mg, mh};
}

// The same evaluation for data with many narrow features: one block handles a chunk of whole features whose bins
// add up to at most 256 (a 100k-column one-hot-like data set has one or two bins per feature; a block per feature
// would launch millions of near-empty blocks).  The scan is segmented by feature; the record of a (node, chunk) keeps
// the GLOBAL bin index of its best candidate.  grid = (chunks, pairs); block = 64.
template <typename T>
static __global__ void __launch_bounds__(64)
k_eval_chunk(int level, int n_chunks, int B, const int *__restrict__ chunk_bin0, const int *__restrict__ cut_ptr,
             const int *__restrict__ cut_fid, const TreeNode *__restrict__ nodes, const int *__restrict__ built_right,
             const T *__restrict__ built, const T *__restrict__ parent, T *__restrict__ full,
             const QuantInfo *__restrict__ q, float mcw, float lam, SplitRec *__restrict__ recs, int bs,
             const unsigned char *__restrict__ ignored_all, const RoundState *__restrict__ rs, int F, int multi) {
    __shared__ T sg[2][256], sh[2][256];
    const unsigned char *ignored = ignored_all ? ignored_all + (size_t)rs->round * F : nullptr;
    const int c = blockIdx.x, j = blockIdx.y;
    const int b0 = chunk_bin0[c], nb = chunk_bin0[c + 1] - b0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_children = level == 0 ? 1 : 2;
    const int node_local = level == 0 ? 0 : 2 * j + warp;
    const int off = (1 << level) - 1;
    const SplitRec none = {0.f, -1, 0.f, 0.f, 0.f, 0.f};
    const int br = built_right[j];
    if (nb == 0 || br < 0) {
        if (lane == 0 && warp < n_children) recs[(size_t)node_local * n_chunks + c] = none;
        return;
    }
    if (level == 0) {
        for (int i = threadIdx.x; i < nb; i += 64) {
            const T cg = built[(size_t)2 * bs * (b0 + i)], ch = built[(size_t)2 * bs * (b0 + i) + 1];
            sg[0][i] = cg; sh[0][i] = ch;
            if (bs != 1) { full[2 * (b0 + i)] = cg; full[2 * (b0 + i) + 1] = ch; }
        }
    } else {
        const T *bp = built + (size_t)j * B * 2 * bs, *pp = parent + (size_t)j * B * 2;
        T *fb = full + (size_t)(2 * j + br) * B * 2, *fo = full + (size_t)(2 * j + 1 - br) * B * 2;
        for (int i = threadIdx.x; i < nb; i += 64) {
            const T cg = bp[(size_t)2 * bs * (b0 + i)], ch = bp[(size_t)2 * bs * (b0 + i) + 1];
            const T og = pp[2 * (b0 + i)] - cg, oh = pp[2 * (b0 + i) + 1] - ch;
            sg[br][i] = cg; sh[br][i] = ch;
            sg[1 - br][i] = og; sh[1 - br][i] = oh;
            fb[2 * (b0 + i)] = cg; fb[2 * (b0 + i) + 1] = ch;
            fo[2 * (b0 + i)] = og; fo[2 * (b0 + i) + 1] = oh;
        }
    }
    __syncthreads();
    if (warp >= n_children) return;
    const TreeNode nd = nodes[off + node_local];
    if (!nd.is_valid) {
        if (lane == 0) recs[(size_t)node_local * n_chunks + c] = none;
        return;
    }
    // lane-local pass over 8 consecutive bins; sums restart where a feature starts
    T eg[8], eh[8];       // exclusive prefix inside the feature, as far as the lane can see
    bool before_start[8];         // no feature start in this lane up to and including this bin -> add the carry
    T rg = 0, rh = 0;
    bool seen = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int b = lane * 8 + i;
        if (b < nb) {
            const int f = cut_fid[b0 + b];
            if (cut_ptr[f] == b0 + b) { rg = 0; rh = 0; seen = true; }
            eg[i] = rg; eh[i] = rh; before_start[i] = !seen;
            rg += sg[warp][b]; rh += sh[warp][b];
        } else { eg[i] = 0; eh[i] = 0; before_start[i] = false; }
    }
    // segmented inclusive scan of the lanes' open tails (rg, rh); flag = the lane contains a feature start
    T vg = rg, vh = rh;
    bool fl = seen;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T ug = shfl_up_t(vg, o), uh = shfl_up_t(vh, o);
        const int uf = __shfl_up_sync(0xffffffffu, (int)fl, o);
        if (lane >= o) {
            if (!fl) { vg += ug; vh += uh; }
            fl = fl || uf;
        }
    }
    T cg = shfl_up_t(vg, 1), ch = shfl_up_t(vh, 1);  // carry into this lane = inclusive value of lane-1
    if (lane == 0) { cg = 0; ch = 0; }
    // inclusive prefix per bin back into shared memory: the last bin of a feature then holds the feature total
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int b = lane * 8 + i;
        if (b < nb) {
            if (before_start[i]) { eg[i] += cg; eh[i] += ch; }
            const T ig = eg[i] + sg[warp][b], ih = eh[i] + sh[warp][b];
            sg[warp][b] = ig; sh[warp][b] = ih;
        }
    }
    __syncwarp();
    const float pg = nd.sum_g, ph = nd.sum_h;
    const double inv_sg = cell_inv<T>(q, 0), inv_sh = cell_inv<T>(q, 1);
    float best = 0.f, best_lg = 0.f, best_lh = 0.f, best_mg = 0.f, best_mh = 0.f;
    int best_bin = -1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int b = lane * 8 + i;
        if (b < nb && !(ignored && ignored[cut_fid[b0 + b]])) {
            const int f = cut_fid[b0 + b];
            const int lastb = cut_ptr[f + 1] - 1 - b0;
            const float mg = __fsub_rn(pg, cell_f(sg[warp][lastb], inv_sg)), mh = __fsub_rn(ph, cell_f(sh[warp][lastb], inv_sh));
            float gn, keep_g, keep_h;
            if (multi) {  // inclusive prefix = right child, see eval_feature
                const float rg = cell_f(sg[warp][b], inv_sg), rh = cell_f(sh[warp][b], inv_sh);
                const float gl = fmaxf(0.f, split_gain(pg, ph, __fsub_rn(pg, rg), __fsub_rn(ph, rh), rg, rh, mcw, lam));
                const float rg2 = __fadd_rn(rg, mg), rh2 = __fadd_rn(rh, mh);
                const float gr = fmaxf(0.f, split_gain(pg, ph, __fsub_rn(pg, rg2), __fsub_rn(ph, rh2), rg2, rh2, mcw, lam));
                gn = gl > gr ? gl : -gr; keep_g = rg; keep_h = rh;
            } else {
                const float lg = cell_f(eg[i], inv_sg), lh = cell_f(eh[i], inv_sh);
                const float gr = fmaxf(0.f, split_gain(pg, ph, lg, lh, __fsub_rn(pg, lg), __fsub_rn(ph, lh), mcw, lam));
                const float lg2 = __fadd_rn(lg, mg), lh2 = __fadd_rn(lh, mh);
                const float gl = fmaxf(0.f, split_gain(pg, ph, lg2, lh2, __fsub_rn(pg, lg2), __fsub_rn(ph, lh2), mcw, lam));
                gn = gl > gr ? gl : -gr; keep_g = lg; keep_h = lh;
            }
            if (best_bin < 0 || fabsf(gn) > fabsf(best)) { best = gn; best_bin = b0 + b; best_lg = keep_g; best_lh = keep_h; best_mg = mg; best_mh = mh; }
        }
    }
    unsigned long long key = best_bin < 0 ? 0ull
                                          : (((unsigned long long)__float_as_uint(fabsf(best)) << 32) | (unsigned)(0x7fffffff - best_bin));
    unsigned long long mk = key;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = (unsigned long long)shfl_xor_ll((long long)mk, o);
        mk = other > mk ? other : mk;
    }
    const unsigned win = __ballot_sync(0xffffffffu, key == mk && best_bin >= 0);
    const int src = __ffs(win) - 1;
    best = __shfl_sync(0xffffffffu, best, src);
    best_bin = __shfl_sync(0xffffffffu, best_bin, src);
    best_lg = __shfl_sync(0xffffffffu, best_lg, src);
    best_lh = __shfl_sync(0xffffffffu, best_lh, src);
    best_mg = __shfl_sync(0xffffffffu, best_mg, src);
    best_mh = __shfl_sync(0xffffffffu, best_mh, src);
    if (lane == 0) recs[(size_t)node_local * n_chunks + c] = SplitRec{best, best_bin, best_lg, best_lh, best_mg, best_mh};
}

// Per-node argmax over the features, SplitPoint decode and update_tree
// (hist_tree_builder_single.cu:365-389 and :847-902).  Called by one whole warp for node n of the level.  The records
// may have been written by other blocks of the running kernel: they are read past L1.
__device__ __forceinline__ SplitRec load_rec(const SplitRec *p) {
    SplitRec r;
    r.gain = __ldcg(&p->gain); r.bin = __ldcg(&p->bin);
    r.lg = __ldcg(&p->lg); r.lh = __ldcg(&p->lh); r.mg = __ldcg(&p->mg); r.mh = __ldcg(&p->mh);
    return r;
}
__device__ __forceinline__ void best_apply_node(int level, int n, int F, const int *__restrict__ cut_ptr,
                                                const float *__restrict__ cut_val, const SplitRec *recs, TreeNode *nodes,
                                                float rt_eps, float lam, const int *__restrict__ cut_fid, int chunked, int multi) {
    // chunked: F is the number of chunks and a record's bin is a global bin index (k_eval_chunk);
    // otherwise one record per feature with a feature-local bin (k_eval).  Ties go to the smaller global bin either way.
    const int lane = threadIdx.x & 31;
    const int nid = (1 << level) - 1 + n;
    if (!nodes[nid].is_valid) return;
    unsigned long long key = 0;
    int key_col = 0;  // record column (feature or chunk) of this lane's best key
    for (int f = lane; f < F; f += 32) {
        const SplitRec r = load_rec(recs + (size_t)n * F + f);
        if (r.bin < 0) continue;
        const unsigned long long k = ((unsigned long long)__float_as_uint(fabsf(r.gain)) << 32) |
                                     (unsigned)(0x7fffffff - (chunked ? r.bin : f));
        if (k > key) { key = k; key_col = f; }
    }
    // a record with gain 0 still has a key > 0, so 0 means "no record"
    unsigned long long mk = key;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = (unsigned long long)shfl_xor_ll((long long)mk, o);
        mk = other > mk ? other : mk;
    }
    const unsigned winners = __ballot_sync(0xffffffffu, key == mk);
    const int win_col = __shfl_sync(0xffffffffu, key_col, __ffs(winners) - 1);
    if (lane != 0) return;
    TreeNode &nd = nodes[nid];
    if (mk == 0) {  // no feature has a cut point: nothing to split on
        nd.is_leaf = 1;
        nodes[nd.lch_index].is_valid = 0;
        nodes[nd.rch_index].is_valid = 0;
        return;
    }
    int f = 0x7fffffff - (int)(mk & 0xffffffffull);
    SplitRec r;
    if (chunked) {
        const int gbin = f;
        f = cut_fid[gbin];
        r = load_rec(recs + (size_t)n * F + win_col);
        r.bin = gbin - cut_ptr[f];
    } else {
        r = load_rec(recs + (size_t)n * F + f);
    }
    const float gain = fabsf(r.gain);
    if (gain > rt_eps) {
        const bool default_right = r.gain < 0.f;
        const int b0 = cut_ptr[f];
        nd.gain = gain;
        nd.split_feature_id = f;
        nd.split_bid = (unsigned char)r.bin;
        if (multi) {
            // TreeBuilder::update_tree of the column-sharded builder (tree_builder.cu:9-60): the split value is the
            // cut point itself, the record's sums are the right child's, the left child is the node minus it
            nd.split_value = cut_val[b0 + r.bin];
            TreeNode &l = nodes[nd.lch_index], &rc = nodes[nd.rch_index];
            l.is_valid = 1; rc.is_valid = 1;
            float rgs = r.lg, rhs = r.lh;
            if (default_right) { rgs = __fadd_rn(rgs, r.mg); rhs = __fadd_rn(rhs, r.mh); nd.default_right = 1; }
            else nd.default_right = 0;
            rc.sum_g = rgs; rc.sum_h = rhs;
            l.sum_g = __fsub_rn(nd.sum_g, rgs); l.sum_h = __fsub_rn(nd.sum_h, rhs);
            l.base_weight = __fdiv_rn(-l.sum_g, __fadd_rn(l.sum_h, lam));
            rc.base_weight = __fdiv_rn(-rc.sum_g, __fadd_rn(rc.sum_h, lam));
            return;
        }
        if (r.bin == 0) {
            const float c = cut_val[b0];
            nd.split_value = (float)((double)__fsub_rn(c, fabsf(c)) - 1e-5);
        } else {
            nd.split_value = cut_val[b0 + r.bin - 1];
        }
        TreeNode &l = nodes[nd.lch_index], &rc = nodes[nd.rch_index];
        l.is_valid = 1; rc.is_valid = 1;
        float lgs = r.lg, lhs = r.lh;
        if (!default_right) { lgs = __fadd_rn(lgs, r.mg); lhs = __fadd_rn(lhs, r.mh); nd.default_right = 0; }
        else nd.default_right = 1;
        l.sum_g = lgs; l.sum_h = lhs;
        rc.sum_g = __fsub_rn(nd.sum_g, lgs); rc.sum_h = __fsub_rn(nd.sum_h, lhs);
        l.base_weight = __fdiv_rn(-l.sum_g, __fadd_rn(l.sum_h, lam));
        rc.base_weight = __fdiv_rn(-rc.sum_g, __fadd_rn(rc.sum_h, lam));
    } else {
        nd.is_leaf = 1;
        nodes[nd.lch_index].is_valid = 0;
        nodes[nd.rch_index].is_valid = 0;
    }
}

// CSR layout: one warp per node of the level, after k_eval_chunk
static __global__ void __launch_bounds__(32)
k_best_apply(int level, int F, const int *__restrict__ cut_ptr, const float *__restrict__ cut_val,
             const SplitRec *__restrict__ recs, TreeNode *__restrict__ nodes, float rt_eps, float lam,
             const int *__restrict__ cut_fid, int chunked, int multi) {
    best_apply_node(level, blockIdx.x, F, cut_ptr, cut_val, recs, nodes, rt_eps, lam, cut_fid, chunked, multi);
}

// Dense layout: evaluation of every (pair, feature) and, by the block that finishes a pair last, the choice among the
// features and the tree update of the pair's two nodes -- one launch per level instead of two.
// `ticket[pair]` counts the finished blocks of a pair and is left at zero.
template <typename T>
static __global__ void __launch_bounds__(64)
k_eval(int level, int F, int B, const int *__restrict__ cut_ptr, TreeNode *nodes, const int *__restrict__ built_right,
       const T *__restrict__ built, const T *__restrict__ parent, T *__restrict__ full,
       const QuantInfo *__restrict__ q, float mcw, float lam, SplitRec *recs, const float *__restrict__ cut_val,
       float rt_eps, const int *__restrict__ cut_fid, int *__restrict__ ticket, int built_stride,
       const unsigned char *__restrict__ ignored_all, const RoundState *__restrict__ rs, int multi) {
    const unsigned char *ignored = ignored_all ? ignored_all + (size_t)rs->round * F : nullptr;
    eval_feature<T>(level, F, B, cut_ptr, nodes, built_right, built, parent, full, q, mcw, lam, recs, built_stride, ignored, multi);
    __shared__ int last;
    __threadfence();  // the block's records are visible before its ticket is
    __syncthreads();
    if (threadIdx.x == 0) {
        last = atomicAdd(&ticket[blockIdx.y], 1) == (int)gridDim.x - 1;
        if (last) ticket[blockIdx.y] = 0;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    const int warp = threadIdx.x >> 5;
    if (level == 0) { if (warp == 0) best_apply_node(0, 0, F, cut_ptr, cut_val, recs, nodes, rt_eps, lam, cut_fid, 0, multi); }
    else best_apply_node(level, 2 * blockIdx.y + warp, F, cut_ptr, cut_val, recs, nodes, rt_eps, lam, cut_fid, 0, multi);
}

// ------------------------------------------------------------------ instance partition
// (replaces update_ins2node_id + the per-level radix sort, hist_tree_builder_single.cu:908-1020, :397-415)
// Every node of the level that holds records gets ceil(count / PART_TILE) tiles of PART_TILE records;
// node_tile0[n] is the first tile of node n, tile_node[t] the node of tile t (looked up here, off the critical path,
// so that the partition kernels do not search for it tile after tile).  Called by every thread of a 1024-thread block.
__device__ inline int tile_owner(const int *__restrict__ node_tile0, int nl, int t);
__device__ inline void part_plan(int level, const int *__restrict__ seg_cnt, int *__restrict__ node_tile0,
                                 int *__restrict__ tile_node, TreeCtl *__restrict__ ctl, bool count_rows, int *__restrict__ part_base,
                                 int *__restrict__ child_begin, int *__restrict__ child_cnt,
                                 unsigned long long *__restrict__ group_sum, int n_group_words) {
    __shared__ int scratch[33];
    __shared__ unsigned long long rows;
    const int nl = 1 << level;
    // single-pass partition: where the children of node n go in the two output halves = records of the nodes before it;
    // a node without records has no tile that could write its children's (empty) segments
    block_scan_excl(nl, [&](int n) { return seg_cnt[n]; },
                    [&](int n, int b) {
                        part_base[n] = b;
                        if (seg_cnt[n] == 0 && child_cnt) { child_cnt[2 * n] = 0; child_cnt[2 * n + 1] = 0; child_begin[2 * n] = b; child_begin[2 * n + 1] = b; }
                    }, scratch);
    if (threadIdx.x == 0) { ctl->part_ticket = 0; ctl->part_epoch = (ctl->part_epoch + 1) & 0x3fffffffu; }
    if (group_sum)
        for (int g = threadIdx.x; g < n_group_words; g += 1024) group_sum[g] = 0;
    if (threadIdx.x == 0) rows = 0;
    __syncthreads();
    const int total = block_scan_excl(nl, [&](int n) { return (seg_cnt[n] + PART_TILE - 1) / PART_TILE; },
                                      [&](int n, int t0) {
                                          node_tile0[n] = t0;
                                          if (seg_cnt[n]) atomicAdd(&rows, (unsigned long long)seg_cnt[n]);
                                      }, scratch);
    if (threadIdx.x == 0) {
        node_tile0[nl] = total;
        ctl->n_part_tiles[level & 1] = total;
        if (count_rows) ctl->stat_part_rows += rows;  // the last level is not partitioned (k_predict_walk)
    }
    __syncthreads();
    for (int t = threadIdx.x; t < total; t += 1024) tile_node[t] = tile_owner(node_tile0, nl, t);
}

// node that owns tile t: the n with node_tile0[n] <= t < node_tile0[n + 1]
__device__ inline int tile_owner(const int *__restrict__ node_tile0, int nl, int t) {
    int lo = 0, hi = nl;  // first n with node_tile0[n] > t
    while (lo < hi) {
        const int mid = (lo + hi) / 2;
        if (node_tile0[mid] > t) hi = mid; else lo = mid + 1;
    }
    return lo - 1;
}

// Direction of every record of a splittable node: left unless (missing and default right) or
// bin >= split_bid (hist_tree_builder_single.cu:1003-1012).  One bit per record, one count per tile.
// Persistent blocks; a thread handles PART_RPT records of a tile so that their loads overlap.
// SPARSE: the row's bin of the split feature is searched in its CSR bin ids (hist_tree_builder_single.cu:941-966)
// instead of being read from the column-major matrix.
template <bool SPARSE>
static __global__ void __launch_bounds__(PART_THREADS)
k_part_count(int level, const TreeNode *__restrict__ nodes, const int *__restrict__ seg_begin, const int *__restrict__ seg_cnt,
             const int *__restrict__ node_tile0, const TreeCtl *__restrict__ ctl, const int *__restrict__ rec_idx,
             const unsigned char *__restrict__ binsT, size_t Npad, const int *__restrict__ sp_row_ptr,
             const int *__restrict__ sp_bin, const int *__restrict__ cut_ptr, unsigned *__restrict__ bits,
             int *__restrict__ tile_left, const int *__restrict__ tile_node, int rev) {
    __shared__ int wsum[32];
    const int nt = ctl->n_part_tiles[level & 1], nl = 1 << level;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = blockIdx.x; t < nt; t += gridDim.x) {
        __syncthreads();  // wsum of the previous tile has been read
        const int n = tile_node[t];
        const TreeNode nd = nodes[nl - 1 + n];
        if (!(nd.is_valid && !nd.is_leaf)) { if (threadIdx.x == 0) tile_left[t] = 0; continue; }
        const int p0 = seg_begin[n] + (t - node_tile0[n]) * PART_TILE, end = seg_begin[n] + seg_cnt[n];
        const unsigned char *colp = SPARSE ? nullptr : binsT + (size_t)nd.split_feature_id * Npad;
        int r[PART_RPT];
#pragma unroll
        for (int j = 0; j < PART_RPT; ++j) {
            const int p = p0 + j * PART_THREADS + threadIdx.x;
            r[j] = p < end ? (rec_idx ? rec_idx[p] : p) : -1;
        }
        unsigned char b[PART_RPT];
        if (SPARSE) {
            const int c0 = cut_ptr[nd.split_feature_id], c1 = cut_ptr[nd.split_feature_id + 1];
#pragma unroll
            for (int j = 0; j < PART_RPT; ++j) {
                b[j] = MISSING_BIN;
                if (r[j] >= 0) {
                    int lo = sp_row_ptr[r[j]], hi = sp_row_ptr[r[j] + 1];  // bin ids ascend inside a row
                    while (lo < hi) {
                        const int mid = lo + (hi - lo) / 2, v = sp_bin[mid];
                        if (v >= c0 && v < c1) { b[j] = (unsigned char)(v - c0); break; }
                        if (v < c0) lo = mid + 1; else hi = mid;
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < PART_RPT; ++j) b[j] = r[j] >= 0 ? colp[r[j]] : 0;
        }
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < PART_RPT; ++j) {
            const bool left = r[j] >= 0 && ((b[j] == MISSING_BIN) ? !nd.default_right : (rev ? b[j] > nd.split_bid : b[j] < nd.split_bid));
            const unsigned m = __ballot_sync(0xffffffffu, left);
            if (lane == 0) { bits[(size_t)t * (PART_TILE / 32) + j * (PART_THREADS / 32) + warp] = m; cnt += __popc(m); }
        }
        if (lane == 0) wsum[warp] = cnt;
        __syncthreads();
        if (warp == 0) {
            int v = lane < PART_THREADS / 32 ? wsum[lane] : 0;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) tile_left[t] = v;
        }
    }
}

// Prefix of the left counts over the tiles of every node and the child segment table of the next level.
// Rows of nodes that stopped splitting simply drop out of the record lists.  One block of 1024 threads.
static __global__ void __launch_bounds__(1024)
k_part_scan(int level, const TreeNode *__restrict__ nodes, const int *__restrict__ seg_cnt,
            const int *__restrict__ node_tile0, int *__restrict__ tile_left, int *__restrict__ next_begin,
            int *__restrict__ next_cnt, int *__restrict__ gcnt, TreeCtl *__restrict__ ctl) {
    __shared__ int scratch[33];
    const int nt = ctl->n_part_tiles[level & 1], nl = 1 << level;
    // tile_left becomes the inclusive prefix over all tiles
    block_scan_excl(nt, [&](int i) { return tile_left[i]; }, [&](int i, int excl) { tile_left[i] += excl; }, scratch);
    auto splittable = [&](int n) { const TreeNode &nd = nodes[nl - 1 + n]; return nd.is_valid && !nd.is_leaf; };
    for (int n = threadIdx.x; n < nl; n += 1024) {
        int cl = 0, cr = 0;
        if (splittable(n) && seg_cnt[n] > 0) {
            const int t0 = node_tile0[n], t1 = node_tile0[n + 1];
            cl = tile_left[t1 - 1] - (t0 > 0 ? tile_left[t0 - 1] : 0);
            cr = seg_cnt[n] - cl;
        }
        next_cnt[2 * n] = cl; next_cnt[2 * n + 1] = cr;
        gcnt[2 * n] = cl; gcnt[2 * n + 1] = cr;
    }
    __syncthreads();
    const int alive = block_scan_excl(2 * nl, [&](int c) { return next_cnt[c]; }, [&](int c, int pos) { next_begin[c] = pos; }, scratch);
    if (threadIdx.x == 0) ctl->n_records = alive;
}

// Work lists of the next level (which sibling to build, tile sequences, partition tiles), from the child segment
// table k_part_scan left.  Nothing in the scatter of the current level needs them, so the host launches this on a
// second stream beside the scatter.  One block of 1024 threads.
static __global__ void __launch_bounds__(1024)
k_plan_next(int level, const int *__restrict__ next_begin, const int *__restrict__ next_cnt, const int *__restrict__ gcnt,
            const TreeNode *__restrict__ nodes, TreeCtl *__restrict__ ctl, int by_hessian, int *__restrict__ built_right,
            HistWork *__restrict__ work, int *__restrict__ hist_tile_base, int *__restrict__ next_node_tile0, int n_ctas,
            int *__restrict__ cta_off, int4 *__restrict__ seq, int depth, int *__restrict__ next_tile_node, int *__restrict__ part_base,
            int *__restrict__ child_begin, int *__restrict__ child_cnt, unsigned long long *__restrict__ group_sum, int n_group_words) {
    // child_begin / child_cnt: segment table of level + 2, the one the partition of level + 1 will fill
    hist_plan(level + 1, next_begin, next_cnt, gcnt, nodes, by_hessian, built_right, work, hist_tile_base, ctl, n_ctas, cta_off, seq);
    __syncthreads();
    part_plan(level + 1, next_cnt, next_node_tile0, next_tile_node, ctl, level + 1 < depth - 1, part_base, child_begin, child_cnt,
              group_sum, n_group_words);
}

// work lists of level 0 (the whole data set in the root)
static __global__ void __launch_bounds__(1024)
k_plan_root(const int *__restrict__ seg_begin, const int *__restrict__ seg_cnt, const int *__restrict__ gcnt,
            const TreeNode *__restrict__ nodes, int *__restrict__ built_right, HistWork *__restrict__ work,
            int *__restrict__ hist_tile_base, int *__restrict__ node_tile0, TreeCtl *__restrict__ ctl, int n_ctas, int *__restrict__ cta_off,
            int4 *__restrict__ seq, int depth, int *__restrict__ tile_node, int *__restrict__ part_base,
            int *__restrict__ child_begin, int *__restrict__ child_cnt, unsigned long long *__restrict__ group_sum, int n_group_words) {
    hist_plan(0, seg_begin, seg_cnt, gcnt, nodes, 0, built_right, work, hist_tile_base, ctl, n_ctas, cta_off, seq);
    __syncthreads();
    part_plan(0, seg_cnt, node_tile0, tile_node, ctl, depth > 1, part_base, child_begin, child_cnt, group_sum, n_group_words);
}

// Stable scatter of the records into the child segments; records of nodes that stopped splitting are dropped.
static __global__ void __launch_bounds__(PART_THREADS)
k_part_scatter(int level, const TreeNode *__restrict__ nodes, const int *__restrict__ seg_begin,
               const int *__restrict__ seg_cnt, const int *__restrict__ node_tile0, const TreeCtl *__restrict__ ctl,
               const int *__restrict__ rec_idx, const int2 *__restrict__ rec_gh, const unsigned *__restrict__ bits,
               const int *__restrict__ tile_left, const int *__restrict__ next_begin,
               int *__restrict__ out_idx, int2 *__restrict__ out_gh, const int *__restrict__ tile_node) {
    constexpr int WORDS = PART_TILE / 32;
    __shared__ int wpre[WORDS];
    __shared__ int wtot[(WORDS + 31) / 32];
    const int nt = ctl->n_part_tiles[level & 1], nl = 1 << level;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = blockIdx.x; t < nt; t += gridDim.x) {
        __syncthreads();  // wpre / wtot of the previous tile have been read
        const int n = tile_node[t];
        const TreeNode nd = nodes[nl - 1 + n];
        const int b = seg_begin[n], end = b + seg_cnt[n];
        const int t0 = node_tile0[n];
        const int p0 = b + (t - t0) * PART_TILE;
        if (!(nd.is_valid && !nd.is_leaf)) continue;  // finished node
        // loads first, so that they overlap with the rank computation
        int r[PART_RPT];
        int2 g[PART_RPT];
        unsigned m[PART_RPT];
#pragma unroll
        for (int j = 0; j < PART_RPT; ++j) {
            const int p = p0 + j * PART_THREADS + threadIdx.x;
            r[j] = p < end ? (rec_idx ? rec_idx[p] : p) : -1;
            if (p < end) g[j] = rec_gh[p];
            m[j] = bits[(size_t)t * WORDS + j * (PART_THREADS / 32) + warp];
        }
        // exclusive prefix of the left counts over the tile's ballot words (record order = word order)
        if (threadIdx.x < WORDS) {
            const int c = __popc(bits[(size_t)t * WORDS + threadIdx.x]);
            int v = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
            wpre[threadIdx.x] = v - c;
            if (lane == 31) wtot[warp] = v;
        }
        __syncthreads();
        const int node_l0 = t0 > 0 ? tile_left[t0 - 1] : 0;
        const int lefts_before_tile = (t > 0 ? tile_left[t - 1] : 0) - node_l0;
#pragma unroll
        for (int j = 0; j < PART_RPT; ++j) {
            if (r[j] < 0) continue;
            const int p = p0 + j * PART_THREADS + threadIdx.x;
            const int w = j * (PART_THREADS / 32) + warp;
            int pre = wpre[w];
            for (int q = 0; q < (w >> 5); ++q) pre += wtot[q];
            const bool left = (m[j] >> lane) & 1u;
            const int lefts_before = lefts_before_tile + pre + __popc(m[j] & ((1u << lane) - 1u));
            const int rank = left ? lefts_before : (p - b) - lefts_before;
            const int d = (left ? next_begin[2 * n] : next_begin[2 * n + 1]) + rank;
            out_idx[d] = r[j];
            out_gh[d] = g[j];
        }
    }
}


// ---- the same in one pass ----------------------------------------------------------------------------------------
// Count, prefix and scatter of a level in ONE kernel.  The output list has two halves: the left children of all nodes
// go to the first half, the right children to the second, both at offset part_base[n] = records of the nodes before
// node n.  A record's place then depends only on how many records BEFORE it in its own node go left -- a prefix
// inside the node.  Every tile publishes its own left count as soon as it has it, per tile and summed per aligned
// group of 32 tiles; a tile adds up the counts before it from those words (no chain of prefixes: with ~600 tiles in
// flight a chained look-back walks back over all of them).  Tiles are handed out in ascending order by a ticket, so
// a tile only ever waits for tiles that are already running.
// The waits are bounded: a tile that gives up records itself in ctl->error and goes on (the host checks the word
// after its next sync), so no GPU is ever left spinning.
// Stable: the rows of either child ascend like those of the node.  Records of nodes that stopped splitting drop out.
constexpr unsigned long long PART_AGG = 1ull << 32, PART_PREFIX = 2ull << 32;  // kind of a status word (bits 32-33)
constexpr int PART_WAIT_LIMIT = 1 << 22;  // polls of ~50 ns each

__device__ __forceinline__ unsigned long long part_status_wait(const unsigned long long *p, unsigned epoch, TreeCtl *ctl, int tile) {
    for (int it = 0; it < PART_WAIT_LIMIT; ++it) {
        const unsigned long long s = *reinterpret_cast<const volatile unsigned long long *>(p);
        if ((unsigned)(s >> 34) == epoch) return s;
        __nanosleep(40);
    }
    atomicCAS(&ctl->error, 0, 1 + tile);
    return ((unsigned long long)epoch << 34) | PART_PREFIX;  // acts as "nothing before": the result is wrong, the error word says so
}

template <bool SPARSE>
static __global__ void __launch_bounds__(PART_THREADS)
k_part_one(int level, const TreeNode *__restrict__ nodes, const int *__restrict__ seg_begin, const int *__restrict__ seg_cnt,
           const int *__restrict__ node_tile0, const int *__restrict__ tile_node, const int *__restrict__ part_base,
           TreeCtl *__restrict__ ctl, const int *__restrict__ rec_idx, const int2 *__restrict__ rec_gh,
           const unsigned char *__restrict__ binsT, size_t Npad, const int *__restrict__ sp_row_ptr,
           const int *__restrict__ sp_bin, const int *__restrict__ cut_ptr, unsigned long long *__restrict__ status,
           unsigned long long *__restrict__ group_sum, int *__restrict__ next_begin, int *__restrict__ next_cnt,
           int *__restrict__ out_idx, int2 *__restrict__ out_gh, int half, int rev) {
    constexpr int WORDS = PART_TILE / 32;        // ballot words of a tile, in record order
    constexpr int WARPS = PART_THREADS / 32;
    __shared__ int s_tile, s_before;
    __shared__ int wpre[WORDS];
    const int nt = ctl->n_part_tiles[level & 1], nl = 1 << level;
    const unsigned epoch = ctl->part_epoch;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (;;) {
        __syncthreads();  // s_tile, s_before, wpre of the previous tile have been read
        if (threadIdx.x == 0) s_tile = atomicAdd(&ctl->part_ticket, 1);
        __syncthreads();
        const int t = s_tile;
        if (t >= nt) break;
        const int n = tile_node[t];
        const TreeNode nd = nodes[nl - 1 + n];
        const int t0 = node_tile0[n], k = t - t0, cnt = seg_cnt[n];
        const int base = part_base[n];
        if (!(nd.is_valid && !nd.is_leaf)) {  // finished node: its rows leave the lists
            if (k == 0 && threadIdx.x == 0) { next_cnt[2 * n] = 0; next_cnt[2 * n + 1] = 0; next_begin[2 * n] = base; next_begin[2 * n + 1] = half + base; }
            continue;
        }
        const int p0 = seg_begin[n] + k * PART_TILE, end = seg_begin[n] + cnt;
        int r[PART_RPT];
        int2 g[PART_RPT];
#pragma unroll
        for (int j = 0; j < PART_RPT; ++j) {
            const int p = p0 + j * PART_THREADS + threadIdx.x;
            r[j] = p < end ? (rec_idx ? rec_idx[p] : p) : -1;
            if (p < end) g[j] = rec_gh[p];
        }
        unsigned char b[PART_RPT];
        if (SPARSE) {
            const int c0 = cut_ptr[nd.split_feature_id], c1 = cut_ptr[nd.split_feature_id + 1];
#pragma unroll
            for (int j = 0; j < PART_RPT; ++j) {
                b[j] = MISSING_BIN;
                if (r[j] >= 0) {
                    int lo = sp_row_ptr[r[j]], hi = sp_row_ptr[r[j] + 1];  // bin ids ascend inside a row
                    while (lo < hi) {
                        const int mid = lo + (hi - lo) / 2, v = sp_bin[mid];
                        if (v >= c0 && v < c1) { b[j] = (unsigned char)(v - c0); break; }
                        if (v < c0) lo = mid + 1; else hi = mid;
                    }
                }
            }
        } else {
            const unsigned char *colp = binsT + (size_t)nd.split_feature_id * Npad;
#pragma unroll
            for (int j = 0; j < PART_RPT; ++j) b[j] = r[j] >= 0 ? colp[r[j]] : 0;
        }
        unsigned m[PART_RPT];
#pragma unroll
        for (int j = 0; j < PART_RPT; ++j) {
            const bool left = r[j] >= 0 && ((b[j] == MISSING_BIN) ? !nd.default_right : (rev ? b[j] > nd.split_bid : b[j] < nd.split_bid));
            m[j] = __ballot_sync(0xffffffffu, left);
            if (lane == 0) wpre[j * WARPS + warp] = __popc(m[j]);
        }
        __syncthreads();
        // exclusive prefix over the tile's ballot words (WORDS = 64: two per lane of warp 0), look-back for the
        // left count of the node's earlier tiles
        if (warp == 0) {
            const int c0 = wpre[2 * lane], c1 = wpre[2 * lane + 1];
            int v = c0 + c1;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
            const int total = __shfl_sync(0xffffffffu, v, 31);
            wpre[2 * lane] = v - c0 - c1;
            wpre[2 * lane + 1] = v - c1;
            // Left records of the node's earlier tiles.  Every tile publishes its own count at once (a status word, and
            // added into the word of its aligned group of 32 tiles), so nothing here waits on a chain: the tiles between
            // the node's first tile and this one are covered by at most two windows of 32 status words (the ragged ends)
            // and the complete groups between them, all read side by side.
            int before = 0;
            const unsigned long long tag = (unsigned long long)epoch << 34;
            if (lane == 0) {
                *reinterpret_cast<volatile unsigned long long *>(status + t) = tag | PART_AGG | (unsigned)total;
                atomicAdd(group_sum + (t >> 5), (1ull << 32) | (unsigned)total);
            }
            if (k > 0) {
                const int gs = (t0 + 31) >> 5, ge = t >> 5;  // complete groups inside the node before t: [gs, ge)
                int part = 0;
                if (gs > ge) {  // the node starts in t's own group
                    const int idx = t0 + lane;
                    if (idx < t) part = (int)(unsigned)(part_status_wait(status + idx, epoch, ctl, t) & 0xffffffffull);
                } else {
                    const int head = t0 + lane, tail = 32 * ge + lane;
                    if (head < 32 * gs) part = (int)(unsigned)(part_status_wait(status + head, epoch, ctl, t) & 0xffffffffull);
                    if (tail < t) part += (int)(unsigned)(part_status_wait(status + tail, epoch, ctl, t) & 0xffffffffull);
                    for (int g = gs + lane; g < ge; g += 32) {
                        unsigned long long w = 0;
                        int it = 0;
                        for (; it < PART_WAIT_LIMIT; ++it) {
                            w = *reinterpret_cast<const volatile unsigned long long *>(group_sum + g);
                            if ((w >> 32) == 32ull) break;  // all 32 tiles of the group have added their count
                            __nanosleep(40);
                        }
                        if (it == PART_WAIT_LIMIT) atomicCAS(&ctl->error, 0, 1 + t);
                        part += (int)(unsigned)(w & 0xffffffffull);
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                before = part;
            }
            if (lane == 0) {
                s_before = before;
                if (t == node_tile0[n + 1] - 1) {  // the node's last tile knows the node's left count
                    next_cnt[2 * n] = before + total; next_cnt[2 * n + 1] = cnt - (before + total);
                    next_begin[2 * n] = base; next_begin[2 * n + 1] = half + base;
                }
            }
        }
        __syncthreads();
        const int before = s_before;
#pragma unroll
        for (int j = 0; j < PART_RPT; ++j) {
            if (r[j] < 0) continue;
            const int q = k * PART_TILE + j * PART_THREADS + threadIdx.x;  // position in the node
            const bool left = (m[j] >> lane) & 1u;
            const int lefts_before = before + wpre[j * WARPS + warp] + __popc(m[j] & ((1u << lane) - 1u));
            const int d = left ? base + lefts_before : half + base + (q - lefts_before);
            out_idx[d] = r[j];
            out_gh[d] = g[j];
        }
    }
}

// ------------------------------------------------------------------ end of tree
// Tree::prune_self / try_prune_leaf / reorder_nid (src/thundergbm/tree.cu:85-128).  The reference walks the
// leaves in index order and climbs while a parent has two leaf children and gain < gamma; the fixed point of that
// walk does not depend on the order, so the levels are processed bottom-up with one thread per node.  One block.
static __global__ void __launch_bounds__(1024)
k_prune(TreeNode *__restrict__ nodes, int n_nodes, int depth, float gamma, int table_in_smem) {
    extern __shared__ __align__(16) unsigned char sm[];
    __shared__ int scratch[33];
    // trees too large for shared memory (depth 12 to 14) are pruned in place in global memory
    TreeNode *sn = table_in_smem ? reinterpret_cast<TreeNode *>(sm) : nodes;
    if (table_in_smem) {
        for (int i = threadIdx.x; i < n_nodes; i += blockDim.x) sn[i] = nodes[i];
        __syncthreads();
    }
    for (int level = depth - 1; level >= 0; --level) {
        const int nl = 1 << level, off = nl - 1;
        for (int n = threadIdx.x; n < nl; n += blockDim.x) {
            TreeNode &p = sn[off + n];
            if (p.is_valid && !p.is_leaf) {
                TreeNode &l = sn[p.lch_index], &r = sn[p.rch_index];
                if (l.is_valid && l.is_leaf && r.is_valid && r.is_leaf && p.gain < gamma) {
                    l.is_pruned = 1; r.is_pruned = 1; p.is_leaf = 1;
                }
            }
        }
        __syncthreads();
    }
    block_scan_excl(n_nodes, [&](int i) { return (sn[i].is_valid && !sn[i].is_pruned) ? 1 : 0; },
                    [&](int i, int id) { if (sn[i].is_valid && !sn[i].is_pruned) sn[i].final_id = id; }, scratch);
    if (table_in_smem)
        for (int i = threadIdx.x; i < n_nodes; i += blockDim.x) nodes[i] = sn[i];
}

// TreeBuilder::predict_in_training (src/thundergbm/builder/tree_builder.cu:62-74); nvcc contracts the
// reference's `y += lr * w` into one fused multiply-add, written out here.
// The reference looks the row's node up in ins2node_id; here every row walks the finished tree on its own bin
// ids instead (the same comparisons the partition made, so the same node), in row order: the bin rows and the
// scores are streamed once, nothing is scattered, and the last level needs no partition at all.
// A node was split iff its children are valid; pruning only marks nodes, so the walk goes on below a pruned
// parent to find the node the reference's table would hold (`nid_out`) while the score takes the weight of the
// deepest node on the path that survived pruning.
// Walk table entry: flags = split bin (bits 0-7) | default right (8) | was split (9) | pruned (10) |
// bins count down, i.e. left means bin > split bin (11; the column-sharded builder's rule, hist_tree_builder.cu:455-459) | feature << 16
struct WalkNode { int flags; float weight; };
struct WalkSpan { int c0, c1; };  // CSR layout: global bins [c0, c1) of the split feature

__device__ __forceinline__ WalkNode walk_node(const TreeNode *__restrict__ nodes, int i, int rev) {
    const TreeNode nd = nodes[i];
    const bool split = nd.is_valid && nd.lch_index >= 0 && nodes[nd.lch_index].is_valid;
    WalkNode w;
    w.flags = (int)nd.split_bid | (nd.default_right ? 0x100 : 0) | (split ? 0x200 : 0) | (nd.is_pruned ? 0x400 : 0) | (rev ? 0x800 : 0) |
              (split ? (int)((unsigned)nd.split_feature_id << 16) : 0);
    w.weight = nd.base_weight;
    return w;
}
__device__ __forceinline__ WalkSpan walk_span(const TreeNode *__restrict__ nodes, const int *__restrict__ cut_ptr, int i) {
    const TreeNode nd = nodes[i];
    const bool split = nd.is_valid && nd.lch_index >= 0 && nodes[nd.lch_index].is_valid;
    const int f = split ? nd.split_feature_id : 0;
    return WalkSpan{cut_ptr[f], cut_ptr[f + 1]};
}

// LAYOUT 0: dense rows of exactly 32 bytes, held in registers (two 16-byte loads per row; the byte of the split
// feature is picked with selects, so that a step costs no memory access); 1: dense rows of any width, one byte load
// per step; 2: CSR of global bin ids, binary search per step (the feature id does not fit the packed flags there).
// `table_in_smem` = 0 for trees too large for shared memory (depth 13 and 14): the nodes are then decoded from global
// memory at every step.
template <int LAYOUT>
static __global__ void __launch_bounds__(256)
k_predict_walk(const TreeNode *__restrict__ nodes, int n_nodes, int table_in_smem, const unsigned char *__restrict__ bins, int Fpad,
               const int *__restrict__ sp_row_ptr, const int *__restrict__ sp_bin, const int *__restrict__ cut_ptr,
               int n, float lr, float *__restrict__ yp, int *__restrict__ nid_out,
               const float *__restrict__ y, int fuse_objective, double *__restrict__ metric_partial,
               unsigned *__restrict__ maxbits, int rev) {
    // fuse_objective >= 0 (a pointwise objective, one tree per round): the same pass adds up the round's training
    // metric (same grid, same order of additions as k_metric_partial) and finds the maxima of the next round's
    // gradients, so that neither needs a pass of its own over y and the scores.
    const bool fuse = fuse_objective >= 0;
    const int fuse_logistic = fuse_objective == REG_LINEAR ? 0 : 1;
    double msum = 0;
    float mg = 0.f, mh = 0.f;
    extern __shared__ __align__(16) unsigned char walk_sm[];
    WalkNode *wn = reinterpret_cast<WalkNode *>(walk_sm);
    WalkSpan *ws = reinterpret_cast<WalkSpan *>(walk_sm + sizeof(WalkNode) * n_nodes);
    if (table_in_smem) {
        for (int i = threadIdx.x; i < n_nodes; i += blockDim.x) {
            wn[i] = walk_node(nodes, i, rev);
            if (LAYOUT == 2) ws[i] = walk_span(nodes, cut_ptr, i);
        }
        __syncthreads();
    }
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
        int lo0 = 0, hi0 = 0;
        uint32_t w[8];
        const unsigned char *row = bins + (size_t)r * Fpad;
        if (LAYOUT == 2) { lo0 = sp_row_ptr[r]; hi0 = sp_row_ptr[r + 1]; }
        if (LAYOUT == 0) {
            const uint4 a = reinterpret_cast<const uint4 *>(row)[0], b = reinterpret_cast<const uint4 *>(row)[1];
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
        int nid = 0;
        float weight = 0.f;
#pragma unroll 1
        for (;;) {
            const WalkNode wk = table_in_smem ? wn[nid] : walk_node(nodes, nid, rev);
            if (!(wk.flags & 0x400)) weight = wk.weight;
            if (!(wk.flags & 0x200)) break;
            int b = MISSING_BIN;
            if (LAYOUT == 2) {
                const WalkSpan sp = table_in_smem ? ws[nid] : walk_span(nodes, cut_ptr, nid);
                int lo = lo0, hi = hi0;
                while (lo < hi) {  // bin ids ascend inside a row
                    const int mid = lo + (hi - lo) / 2, v = sp_bin[mid];
                    if (v >= sp.c0 && v < sp.c1) { b = v - sp.c0; break; }
                    if (v < sp.c0) lo = mid + 1; else hi = mid;
                }
            } else if (LAYOUT == 1) {
                b = row[(unsigned)wk.flags >> 16];
            } else {
                const unsigned f = (unsigned)wk.flags >> 16;
                const uint32_t a0 = (f & 16) ? w[4] : w[0], a1 = (f & 16) ? w[5] : w[1], a2 = (f & 16) ? w[6] : w[2],
                               a3 = (f & 16) ? w[7] : w[3];
                const uint32_t b0 = (f & 8) ? a2 : a0, b1 = (f & 8) ? a3 : a1;
                b = (((f & 4) ? b1 : b0) >> (8 * (f & 3))) & 0xffu;
            }
            const bool left = (b == MISSING_BIN) ? !(wk.flags & 0x100) : ((wk.flags & 0x800) ? b > (wk.flags & 0xff) : b < (wk.flags & 0xff));
            nid = 2 * nid + (left ? 1 : 2);
        }
        if (nid_out) nid_out[r] = nid;
        const float score = __fmaf_rn(lr, weight, yp[r]);
        yp[r] = score;
        if (fuse) {
            const float yr = y[r];
            msum += pointwise_metric_term(fuse_objective, yr, score);
            const float2 v = pointwise_gh(fuse_logistic, yr, score);
            mg = fmaxf(mg, fabsf(v.x)); mh = fmaxf(mh, v.y);
        }
    }
    if (fuse) {
        __shared__ double ws[8];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) msum += __shfl_xor_sync(0xffffffffu, msum, o);
        if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = msum;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += ws[w];
            metric_partial[blockIdx.x] = t;
        }
        track_max(mg, mh, maxbits);
    }
}

// ------------------------------------------------------------------ metrics
// per-block partial sums in a fixed order: RMSE (pointwise_metric.cu:8-22), binary error and
// multi-class accuracy (multiclass_metric.cu:9-46)
static __global__ void k_metric_partial(int objective, const float *__restrict__ y, const float *__restrict__ yp, int n, int K,
                                 double *__restrict__ partial) {
    __shared__ double ws[32];
    double s = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        if (objective == REG_LINEAR || objective == REG_LOGISTIC || objective == BINARY_LOGISTIC) {
            s += pointwise_metric_term(objective, y[i], yp[i]);
        } else {
            int mk = 0;
            float mp = yp[i];
            for (int k = 1; k < K; ++k) { const float v = yp[(size_t)k * n + i]; if (v > mp) { mp = v; mk = k; } }
            s += ((float)mk == y[i]) ? 1.0 : 0.0;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += ws[w];
        partial[blockIdx.x] = t;
    }
}
// one warp: lane l adds partial[l], partial[l+32], ... in that order, then a fixed shuffle tree
static __global__ void k_metric_sum(const double *__restrict__ partial, int nb, double *__restrict__ out) {
    double t = 0;
    for (int i = threadIdx.x; i < nb; i += 32) t += partial[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) *out = t;
}
__device__ __forceinline__ float metric_from_sum(int objective, double s, long long n_total) {
    if (objective == REG_LINEAR || objective == REG_LOGISTIC) return sqrtf((float)s / (float)n_total);
    if (objective == BINARY_LOGISTIC) return 1.0f - (float)(long long)s / (float)n_total;
    if (objective == RANK_PAIRWISE || objective == RANK_NDCG) return (float)(s / (double)n_total);  // mean over the query groups
    return (float)(long long)s / (float)n_total;
}
static __global__ void k_metric_final(int objective, const double *__restrict__ sum, long long n_total, float *__restrict__ out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) *out = metric_from_sum(objective, *sum, n_total);
}

// End of a boosting round: the round's metric (for ranking `sum` and `n_total` are those of the query groups), the round's
// fixed-point grid for the log, and the device round counter moves on.  One thread.
static __global__ void k_round_end(int objective, const double *__restrict__ sum, long long n_total, float *__restrict__ metric,
                                   const QuantInfo *__restrict__ qinfo, QuantInfo *__restrict__ qinfo_log, int log_len,
                                   RoundState *__restrict__ rs) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int r = rs->round;
        if (objective >= 0) metric[r] = metric_from_sum(objective, *sum, n_total);
        if (r < log_len) qinfo_log[r] = *qinfo;
        rs->round = r + 1;
    }
}

// The finished tree into its slot of the model: tree (round * K + k)
static __global__ void k_store_tree(const TreeNode *__restrict__ nodes, TreeNode *__restrict__ model, int n_nodes, int K, int k,
                                    const RoundState *__restrict__ rs) {
    TreeNode *dst = model + ((size_t)rs->round * K + k) * n_nodes;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_nodes; i += gridDim.x * blockDim.x) dst[i] = nodes[i];
}

static __global__ void k_fill(float *p, size_t n, float v) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}

}  // namespace tgbm
