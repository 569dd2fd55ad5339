// The exact tree builder (tree_method = exact; ExactTreeBuilder, src/thundergbm/builder/exact_tree_builder.cu):
// every distinct stored value of a node is a split candidate.  Same level loop, node table, pruning and scores as
// the histogram builder; what differs is the split search and how the rows move.
//
// Data: the stored values by column, largest first (SparseColumns::csr2csc_gpu, sparse_columns.cu:20-93,127), built
// once.  Per level: every entry gets the key `column * nodes_in_level + node of its row` (entries of rows that
// stopped get the largest key), a stable radix sort by that key groups the entries of each (column, node) while
// keeping the values descending, a scan by key gives every entry the (g,h) sum of its group up to itself, and the
// last entry of each run of equal values is a candidate whose right child is that sum (exact_tree_builder.cu:50-118).
#pragma once
#include "tgbm_kernels.cuh"

namespace tgbm {

constexpr unsigned EX_NONE = 0xffffffffu;   // key of an entry whose row is not in a node of the running level
constexpr int EX_THREADS = 512;

template <typename T> struct ExPair { T g, h; };
template <typename T> struct ExAdd {
    __host__ __device__ __forceinline__ ExPair<T> operator()(const ExPair<T> &a, const ExPair<T> &b) const { return ExPair<T>{a.g + b.g, a.h + b.h}; }
};
// sorted position -> (g,h) of the entry's row; the float arithmetic reads the float pair, the fixed-point one the
// quantised pair (both 8 bytes per row)
template <typename T> struct ExGather;
template <> struct ExGather<float> {
    const unsigned *idx; const int *e_row; const float2 *gh;
    __host__ __device__ __forceinline__ ExPair<float> operator()(long long j) const {
        const float2 v = gh[e_row[idx[j]]];
        return ExPair<float>{v.x, v.y};
    }
};
template <> struct ExGather<long long> {
    const unsigned *idx; const int *e_row; const int2 *gh;
    __host__ __device__ __forceinline__ ExPair<long long> operator()(long long j) const {
        const int2 v = gh[e_row[idx[j]]];
        return ExPair<long long>{(long long)v.x, (long long)v.y};
    }
};

// row id of every stored value (CSR order)
static __global__ void k_exact_rows(const int *__restrict__ row_ptr, int n_rows, int *__restrict__ out) {
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x)
        for (int j = row_ptr[r]; j < row_ptr[r + 1]; ++j) out[j] = r;
}
// (column, complement of the value's ordered image): ascending keys = columns ascending, values descending
static __global__ void k_exact_csc_keys(const float *__restrict__ val, const int *__restrict__ col, size_t nnz, unsigned long long *__restrict__ keys) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nnz; i += (size_t)gridDim.x * blockDim.x)
        keys[i] = ((unsigned long long)(unsigned)col[i] << 32) | (unsigned)~float_order(val[i]);
}
static __global__ void k_exact_csc_vals(const unsigned long long *__restrict__ keys, size_t nnz, float *__restrict__ val) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nnz; i += (size_t)gridDim.x * blockDim.x)
        val[i] = order_float(~(unsigned)(keys[i] & 0xffffffffull));
}
static __global__ void k_exact_iota(unsigned *p, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = (unsigned)i;
}

// column of entry i: the f with csc_ptr[f] <= i < csc_ptr[f + 1]
__device__ __forceinline__ int exact_column(const long long *__restrict__ csc_ptr, int F, long long i) {
    int lo = 0, hi = F;   // first f with csc_ptr[f] > i
    while (lo < hi) {
        const int mid = (lo + hi) / 2;
        if (csc_ptr[mid] > i) hi = mid; else lo = mid + 1;
    }
    return lo - 1;
}

// exact_tree_builder.cu:57-76: entry -> partition id (column-major over the nodes of the level)
static __global__ void k_exact_keys(const int *__restrict__ e_row, long long nnz, const long long *__restrict__ csc_ptr, int F,
                                    const int *__restrict__ nid, int level, unsigned *__restrict__ keys) {
    const int nl = 1 << level, off = nl - 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nnz; i += (long long)gridDim.x * blockDim.x) {
        const int n = nid[e_row[i]] - off;
        keys[i] = (n >= 0 && n < nl) ? (unsigned)exact_column(csc_ptr, F, i) * (unsigned)nl + (unsigned)n : EX_NONE;
    }
}

// first sorted position of every partition id (exact_tree_builder.cu:124-127)
static __global__ void k_exact_pid_ptr(const unsigned *__restrict__ keys, long long nnz, long long n_pid, int *__restrict__ pid_ptr) {
    for (long long pid = blockIdx.x * (long long)blockDim.x + threadIdx.x; pid <= n_pid; pid += (long long)gridDim.x * blockDim.x) {
        long long lo = 0, hi = nnz;
        while (lo < hi) {
            const long long mid = lo + (hi - lo) / 2;
            if (keys[mid] < (unsigned)pid) lo = mid + 1; else hi = mid;
        }
        pid_ptr[pid] = (int)lo;
    }
}

template <typename T>
__device__ __forceinline__ float exact_gain(const TreeNode &nd, const ExPair<T> &right, const ExPair<T> &total, double inv_sg, double inv_sh,
                                            float mcw, float lam, float &rg, float &rh, float &mg, float &mh) {
    // exact_tree_builder.cu:160-167 (missing = node sum - sum of the stored values) and :186-209 (gain, default direction)
    const float pg = nd.sum_g, ph = nd.sum_h;
    mg = __fsub_rn(pg, cell_f(total.g, inv_sg)); mh = __fsub_rn(ph, cell_f(total.h, inv_sh));
    rg = cell_f(right.g, inv_sg); rh = cell_f(right.h, inv_sh);
    const float gl = fmaxf(0.f, split_gain(pg, ph, __fsub_rn(pg, rg), __fsub_rn(ph, rh), rg, rh, mcw, lam));
    const float rg2 = __fadd_rn(rg, mg), rh2 = __fadd_rn(rh, mh);
    const float gr = fmaxf(0.f, split_gain(pg, ph, __fsub_rn(pg, rg2), __fsub_rn(ph, rh2), rg2, rh2, mcw, lam));
    return gl > gr ? gl : -gr;
}

// Gain of every candidate and the best one per node: key = |gain| bits << 32 | ~position, so that the largest key is
// the largest |gain| and among equals the smallest sorted position (exact_tree_builder.cu:218-258: smaller partition
// id, i.e. smaller column, then larger value).  Per block the keys meet in shared memory (one slot per node of the
// level), warps whose lanes all sit in one node reduce first.
template <typename T>
static __global__ void __launch_bounds__(EX_THREADS)
k_exact_gain(const unsigned *__restrict__ keys, const unsigned *__restrict__ idx, const float *__restrict__ e_val,
             const ExPair<T> *__restrict__ sums, const int *__restrict__ pid_ptr, long long nnz, int level,
             const TreeNode *__restrict__ nodes, const QuantInfo *__restrict__ q, float mcw, float lam,
             const unsigned char *__restrict__ ignored_all, const RoundState *__restrict__ rs, int F,
             unsigned long long *__restrict__ best) {
    extern __shared__ unsigned long long ex_best[];
    const int nl = 1 << level, off = nl - 1;
    for (int n = threadIdx.x; n < nl; n += blockDim.x) ex_best[n] = 0;
    __syncthreads();
    const unsigned char *ignored = ignored_all ? ignored_all + (size_t)rs->round * F : nullptr;
    const double inv_sg = cell_inv<T>(q, 0), inv_sh = cell_inv<T>(q, 1);
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long rounds = (nnz + stride - 1) / stride;
    for (long long it = 0; it < rounds; ++it) {
        const long long j = it * stride + blockIdx.x * (long long)blockDim.x + threadIdx.x;
        unsigned long long cand = 0;
        int n = -1;
        if (j < nnz) {
            const unsigned key = keys[j];
            if (key != EX_NONE) {
                const int end = pid_ptr[key + 1];
                const bool last_of_run = j + 1 == end || e_val[idx[j + 1]] != e_val[idx[j]];
                if (last_of_run) {
                    n = (int)(key % (unsigned)nl);
                    const int f = (int)(key / (unsigned)nl);
                    float gn = 0.f, rg, rh, mg, mh;
                    if (!(ignored && ignored[f])) gn = exact_gain<T>(nodes[off + n], sums[j], sums[end - 1], inv_sg, inv_sh, mcw, lam, rg, rh, mg, mh);
                    cand = ((unsigned long long)__float_as_uint(fabsf(gn)) << 32) | (unsigned)(0xffffffffu - (unsigned)j);
                }
            }
        }
        // warps in one node (the usual case: the entries of a (column, node) are consecutive) send one key
        const int n0 = __shfl_sync(0xffffffffu, n, 0);
        if (__all_sync(0xffffffffu, n == n0 || n < 0)) {
            const int nn = __reduce_max_sync(0xffffffffu, n);
            unsigned long long mk = cand;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = (unsigned long long)shfl_xor_ll((long long)mk, o);
                mk = other > mk ? other : mk;
            }
            if ((threadIdx.x & 31) == 0 && nn >= 0 && mk) atomicMax(&ex_best[nn], mk);
        } else if (n >= 0) {
            atomicMax(&ex_best[n], cand);
        }
    }
    __syncthreads();
    for (int n = threadIdx.x; n < nl; n += blockDim.x)
        if (ex_best[n]) atomicMax(&best[n], ex_best[n]);
}

// SplitPoint of the best candidate and TreeBuilder::update_tree (exact_tree_builder.cu:262-296, :137-151 for the split
// value; tree_builder.cu:9-60).  One thread per node of the level.
template <typename T>
static __global__ void k_exact_apply(const unsigned *__restrict__ keys, const unsigned *__restrict__ idx, const float *__restrict__ e_val,
                                     const ExPair<T> *__restrict__ sums, const int *__restrict__ pid_ptr, int level,
                                     TreeNode *__restrict__ nodes, const QuantInfo *__restrict__ q, float mcw, float lam, float rt_eps,
                                     unsigned long long *__restrict__ best, int *__restrict__ any_split) {
    const int nl = 1 << level, off = nl - 1;
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n == 0) *any_split = 0;
    if (n >= nl) return;
    const unsigned long long b = best[n];
    best[n] = 0;
    TreeNode &nd = nodes[off + n];
    if (!nd.is_valid || b == 0) return;   // no stored value in the node: SplitPoint::nid = -1, the node stays as it is
    const long long j = (long long)(0xffffffffu - (unsigned)(b & 0xffffffffull));
    const unsigned key = keys[j];
    const int f = (int)(key / (unsigned)nl), begin = pid_ptr[key], end = pid_ptr[key + 1];
    float rg, rh, mg, mh;
    const float gn = exact_gain<T>(nd, sums[j], sums[end - 1], cell_inv<T>(q, 0), cell_inv<T>(q, 1), mcw, lam, rg, rh, mg, mh);
    const float gain = __uint_as_float((unsigned)(b >> 32));   // |gn|, or 0 for a column left out of the round
    if (gain > rt_eps) {
        const float v = e_val[idx[j]];
        nd.gain = gain;
        nd.split_feature_id = f;
        nd.split_bid = 0;
        nd.split_value = j + 1 == end ? __fsub_rn(__fsub_rn(v, fabsf(e_val[idx[begin]])), rt_eps)
                                      : __fmul_rn(__fadd_rn(v, e_val[idx[j + 1]]), 0.5f);
        TreeNode &l = nodes[nd.lch_index], &rc = nodes[nd.rch_index];
        l.is_valid = 1; rc.is_valid = 1;
        float rgs = rg, rhs = rh;
        if (gn < 0.f) { rgs = __fadd_rn(rgs, mg); rhs = __fadd_rn(rhs, mh); nd.default_right = 1; }
        else nd.default_right = 0;
        rc.sum_g = rgs; rc.sum_h = rhs;
        l.sum_g = __fsub_rn(nd.sum_g, rgs); l.sum_h = __fsub_rn(nd.sum_h, rhs);
        l.base_weight = __fdiv_rn(-l.sum_g, __fadd_rn(l.sum_h, lam));
        rc.base_weight = __fdiv_rn(-rc.sum_g, __fadd_rn(rc.sum_h, lam));
    } else {
        nd.is_leaf = 1;
        nodes[nd.lch_index].is_valid = 0;
        nodes[nd.rch_index].is_valid = 0;
    }
}

// ExactTreeBuilder::update_ins2node_id (exact_tree_builder.cu:303-340): a row that stores the split feature of its
// node goes by the value.  The entry of (row, split feature) is the only writer of the row's slot; another entry of
// the row that reads the slot afterwards finds the child, whose split feature is still unset.
static __global__ void k_exact_move(const int *__restrict__ e_row, const float *__restrict__ e_val, long long nnz,
                                    const long long *__restrict__ csc_ptr, int F, int *nid, const TreeNode *__restrict__ nodes,
                                    int *__restrict__ any_split) {
    bool any = false;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nnz; i += (long long)gridDim.x * blockDim.x) {
        const int r = e_row[i];
        const int at = nid[r];
        const TreeNode nd = nodes[at];
        if (nd.is_leaf || !nd.is_valid || nd.split_feature_id < 0) continue;
        if (nd.split_feature_id != exact_column(csc_ptr, F, i)) continue;
        any = true;
        nid[r] = e_val[i] < nd.split_value ? nd.lch_index : nd.rch_index;
    }
    if (__any_sync(0xffffffffu, any) && (threadIdx.x & 31) == 0) *any_split = 1;
}
// ... and ExactTreeBuilder::ins2node_id_all_reduce (:394-409): the rows still in a splittable node of the level follow
// its default direction; skipped when no row moved at this level (tree_builder.cu:174-181 leaves the loop first)
static __global__ void k_exact_move_missing(int *__restrict__ nid, int n_rows, int level, const TreeNode *__restrict__ nodes,
                                            const int *__restrict__ any_split) {
    if (!*any_split) return;
    const int nl = 1 << level, off = nl - 1;
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
        const int at = nid[r];
        if (at < off || at >= off + nl) continue;
        const TreeNode nd = nodes[at];
        if (nd.is_leaf || !nd.is_valid) continue;
        nid[r] = nd.default_right ? nd.rch_index : nd.lch_index;
    }
}

// TreeBuilder::predict_in_training (tree_builder.cu:62-74) from the row -> node table
static __global__ void k_exact_predict(const int *__restrict__ nid, int n_rows, const TreeNode *__restrict__ nodes, float lr,
                                       float *__restrict__ yp, int *__restrict__ nid_out) {
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
        int n = nid[r];
        if (nid_out) nid_out[r] = n;
        while (n != -1 && nodes[n].is_pruned) n = nodes[n].parent_index;
        yp[r] = __fmaf_rn(lr, nodes[n].base_weight, yp[r]);
    }
}

}  // namespace tgbm
