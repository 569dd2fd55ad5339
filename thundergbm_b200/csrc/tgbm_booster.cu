// Host orchestration of the boosting loop: every launch of a round is queued on one stream and
// nothing in boost() waits for the device, so the level loop never round-trips through the host
// (the reference synchronises after every launch, include/thundergbm/util/device_lambda.cuh:49).
#include "tgbm_booster.h"

#include <cub/cub.cuh>
#include <cub/device/device_merge.cuh>
#include <cuda/std/functional>

#include <algorithm>
#include <chrono>
#include <climits>
#include <cmath>
#include <cstddef>
#include <cstdlib>
#include <cstring>

#include "tgbm_kernels.cuh"
#include "tgbm_hist_f32.cuh"
#include "tgbm_exact.cuh"
#include "tgbm_rank.cuh"

namespace tgbm {

struct BoosterImpl {
    GBMParam p;
    const Comm *comm = nullptr;
    cudaStream_t stream = nullptr;
    cudaStream_t stream2 = nullptr;          // side stream for planning kernels that run beside the scatter
    cudaEvent_t ev_scan = nullptr, ev_plan = nullptr;
    int objective = REG_LINEAR;
    int N = 0, F = 0, Fpad = 0, G = 0, B = 0, K = 1, n_nodes = 0, depth = 0;
    long long N_global = 0;
    long long row_offset = 0;  // global id of local row 0
    size_t Npad = 0;
    int num_class = 1;
    float base_score = 0;
    int rounds = 0;
    int num_sms = 148;
    int window_rows = 0;
    bool profile_on = false;

    std::vector<float> h_cut_val;
    std::vector<int> h_cut_ptr;
    std::vector<float> label;

    DevBuf<int> d_row_ptr, d_col;  // the input CSR on the device, held from upload_csr() to the end of binning
    DevBuf<float> d_val;
    DevBuf<unsigned char> bins, binsT;
    // wide sparse data: CSR of global bin ids instead of the two dense matrices
    bool sparse = false;
    long long nnz_local = 0;
    DevBuf<int> sp_row_ptr, sp_bin, chunk_bin0;
    int n_chunks = 0;
    DevBuf<float> cut_val, y, ypred, metric;
    DevBuf<int> cut_ptr, cut_fid;
    DevBuf<float2> gh;
    DevBuf<int2> ghq;
    DevBuf<unsigned> maxbits;
    DevBuf<unsigned long long> root_sum;
    DevBuf<QuantInfo> qinfo, qinfo_log;
    DevBuf<TreeNode> nodes, model;
    DevBuf<int> rec_idx[2];
    DevBuf<int2> rec_gh[2];
    DevBuf<int> seg_begin[2], seg_cnt[2], gcnt;
    DevBuf<int> nid_keep;
    DevBuf<long long> hist_full, hist_built;
    // fp32 mode: the same two buffers hold float pairs; `hist_spread` receives the built histograms, their cells
    // `f32_stride(pairs)` float2 apart (see tgbm_hist_f32.cuh)
    bool f32 = false;
    DevBuf<float2> hist_spread;
    DevBuf<double> sum_partial;
    CutOffsets f32_cuts{};                 // fp32 dense kernel: first bin of every feature, passed by value
    bool f32_staged = true;                // fp32 dense kernel, gather levels: record tiles staged by bulk copies
    DevBuf<int> bag_count;                 // bagging: multiplicity of every gradient entry in the round's bootstrap sample
    DevBuf<unsigned char> ignored_all;     // column sampling: [round][feature] mask of the features left out
    // Distance of two cells of a built histogram, in cells: 32 (one 8-byte cell per 256 bytes) wherever the spread
    // buffer has room.  The L2 performs reductions to cells that share a line one after the other: a microbenchmark of
    // the bare reductions (10.5 M rows x 28) runs at 87 / 165 / 176 / 190 / 165 G/s with 8 / 64 / 128 / 256 / 512 bytes
    // between the cells of one node, and the whole boosting round got 13 % shorter going from 64 to 256 bytes.
    size_t spread_cells = 0;   // float2 cells of hist_spread
    int f32_stride(int pairs) const {
        int s = 32;
        while (s > 1 && (size_t)s * pairs * std::max(B, 1) > spread_cells) s >>= 1;
        return s;
    }
    DevBuf<int> built_right, hist_tile_base;
    DevBuf<HistWork> hist_work;
    bool prune_in_smem = true;
    TreeCtl stat_base{};  // counters of `ctl` when profiling was switched on
    DevBuf<RoundState> rstate;          // device copy of `rounds`
    cudaGraph_t round_graph = nullptr;  // one boosting round (gradients, K trees, metric) as captured in its steady state
    cudaGraphExec_t round_exec = nullptr;
    long long round_graph_launches = 0;
    bool graphs_allowed = true;
    void run_round(int round);
    DevBuf<int> eval_ticket;  // k_eval: finished blocks per sibling pair, zero between launches
    bool grad_max_ready = false;        // maxbits holds the maxima of the next round's gradients
    bool metric_partial_ready = false;  // metric_partial holds the finished round's partial sums
    int metric_blocks() const { return std::max(1, std::min((N + 255) / 256, 1024)); }
    DevBuf<int> hist_cta_off;  // dense histogram kernel: tile sequence of every CTA
    DevBuf<int4> hist_seq;
    DevBuf<SplitRec> recs;
    DevBuf<int> node_tile0[2], tile_left, tile_node[2];
    DevBuf<int> part_base;                    // single-pass partition: records of the nodes before a node
    DevBuf<unsigned long long> part_status;   // single-pass partition: left count of every tile
    DevBuf<unsigned long long> part_group;    // ... and of every aligned group of 32 tiles (count of contributors << 32 | sum)
    bool part_one = false;
    DevBuf<unsigned> bits;
    DevBuf<TreeCtl> ctl;
    DevBuf<double> metric_partial, metric_sum;
    int max_tiles = 0;
    int hist_smem = 0;
    RankState rank;

    struct TimedEvent { cudaEvent_t a, b; int kind; };
    std::vector<TimedEvent> events;
    HistProfile profile_acc;  // kernel times of the events already read and destroyed
    long long launches = 0;

    ~BoosterImpl() {
        if (stream) cudaStreamSynchronize(stream);    // nothing of this booster is in flight when its buffers go
        if (stream2) cudaStreamSynchronize(stream2);
        for (auto &e : events) { cudaEventDestroy(e.a); cudaEventDestroy(e.b); }
        if (round_exec) cudaGraphExecDestroy(round_exec);
        if (round_graph) cudaGraphDestroy(round_graph);
        if (ev_scan) cudaEventDestroy(ev_scan);
        if (ev_plan) cudaEventDestroy(ev_plan);
        if (stream2) cudaStreamDestroy(stream2);
        if (stream) cudaStreamDestroy(stream);
    }

    // ---------------------------------------------------------------- init helpers
    void upload_csr(const DataSet &ds);
    void find_cuts_and_bins(const DataSet &ds);
    // tree_method = exact (tgbm_exact.cuh)
    bool exact = false;
    long long ex_nnz = 0;
    DevBuf<int> ex_row;                 // stored values by column, largest first: row ...
    DevBuf<float> ex_val;               // ... and value
    DevBuf<long long> ex_csc_ptr;
    DevBuf<unsigned> ex_key[2], ex_idx[2];  // per level: partition id of every entry / sorted, entry of every sorted position
    DevBuf<unsigned char> ex_sums;      // ExPair<T> per sorted position: (g,h) of its partition up to itself
    DevBuf<int> ex_pid_ptr, ex_nid, ex_any;
    DevBuf<unsigned long long> ex_best;
    DevBuf<unsigned char> ex_tmp;       // scratch of the radix sort and the scan by key
    void init_exact(const DataSet &ds);
    template <typename T> void exact_levels(int k, const void *gh_rows);
    void build_tree_exact(int round, int k);
    void column_builder_candidates(DevBuf<unsigned long long> &ukeys, DevBuf<long long> &ucopies, long long &nu);
    void init_base_score();
    void gradient(int round);
    void build_tree(int round, int k);
    void round_metric(int round);
    size_t full_offset(int level) const { return ((size_t)(1 << level) - 1) * B * 2; }
};

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Host CSR -> device (asynchronous).  When the caller did not count the features (DataSet::n_features < 0) the largest
// column index is found here, at HBM speed, instead of by a pass over the host copy.
void BoosterImpl::upload_csr(const DataSet &ds) {
    const size_t nnz = (size_t)ds.rp[N];
    d_row_ptr.alloc(N + 1); d_col.alloc(std::max<size_t>(nnz, 1)); d_val.alloc(std::max<size_t>(nnz, 1));
    // host threads that stage a pageable source (fewer per rank when the ranks of one process upload side by side)
    const int up_threads = comm && comm->active() ? std::max(1, upload_threads() / comm->world) : upload_threads();
    upload_h2d(d_row_ptr.p, ds.rp, sizeof(int) * (size_t)(N + 1), stream, up_threads);
    upload_h2d(d_col.p, ds.ci, sizeof(int) * nnz, stream, up_threads);
    upload_h2d(d_val.p, ds.vv, sizeof(float) * nnz, stream, up_threads);
    // Largest and smallest column index, found here at HBM speed: the largest gives the feature count when the caller
    // did not count (dataset.cpp:54-57), a negative one would send the binning kernels out of bounds.
    const bool count_features = F < 0;
    if (count_features) F = 1;
    if (nnz) {
        DevBuf<int> d_mm;
        d_mm.alloc(2);
        size_t tb = 0, tb2 = 0;
        TGBM_CUDA(cub::DeviceReduce::Max(nullptr, tb, d_col.p, d_mm.p, (long long)nnz, stream));
        TGBM_CUDA(cub::DeviceReduce::Min(nullptr, tb2, d_col.p, d_mm.p + 1, (long long)nnz, stream));
        DevBuf<unsigned char> tmp;
        tmp.alloc(std::max<size_t>(std::max(tb, tb2), 1));
        TGBM_CUDA(cub::DeviceReduce::Max(tmp.p, tb, d_col.p, d_mm.p, (long long)nnz, stream));
        TGBM_CUDA(cub::DeviceReduce::Min(tmp.p, tb2, d_col.p, d_mm.p + 1, (long long)nnz, stream));
        int h_mm[2] = {0, 0};
        TGBM_CUDA(cudaMemcpyAsync(h_mm, d_mm.p, sizeof(h_mm), cudaMemcpyDeviceToHost, stream));
        TGBM_CUDA(cudaStreamSynchronize(stream));
        TGBM_CHECK(h_mm[1] >= 0, "negative column index in the CSR input");
        if (count_features) F = h_mm[0] + 1;
        else TGBM_CHECK(h_mm[0] < F, "column index beyond the feature count");
    }
}

// ------------------------------------------------------------------------------------------------
// Cut-point candidates of the reference's column-sharded builder (HistCut::get_cut_points3 + unique_by_flag,
// src/thundergbm/hist_cut.cu:104-187, run by each of its `column_shards` devices on the columns
// SparseColumns::csr2csc_gpu gives it, src/thundergbm/sparse_columns.cu:95-102).  In: the distinct (feature, value)
// keys in ascending order with their multiplicities.  Out: per feature the candidates, largest first, as keys
// (feature, complement of the value's ordered image), from which the usual stride selection picks the cut points.
void BoosterImpl::column_builder_candidates(DevBuf<unsigned long long> &ukeys, DevBuf<long long> &ucopies, long long &nu) {
    if (nu == 0) return;
    const int D = p.column_shards;
    const int grid = std::min(ceil_div(nu, 256), num_sms * 16);
    // copies before every key, per feature the largest value and the copies before its first key
    DevBuf<long long> before, ustart, fbefore;
    DevBuf<float> fmax;
    before.alloc(nu + 1); ustart.alloc(F + 1); fbefore.alloc(F + 1); fmax.alloc(F);
    TGBM_CUDA(cudaMemsetAsync(ucopies.p + nu, 0, sizeof(long long), stream));
    auto scan = [&](const long long *in, long long *out, long long n) {
        size_t tb = 0;
        cub::DeviceScan::ExclusiveSum(nullptr, tb, in, out, n, stream);
        DevBuf<unsigned char> tmp;
        tmp.alloc(std::max<size_t>(tb, 1));
        cub::DeviceScan::ExclusiveSum(tmp.p, tb, in, out, n, stream);
        TGBM_CUDA(cudaStreamSynchronize(stream));
    };
    scan(ucopies.p, before.p, nu + 1);
    long long total = 0;
    TGBM_CUDA(cudaMemcpyAsync(&total, before.p + nu, sizeof(long long), cudaMemcpyDeviceToHost, stream));
    k_feature_bounds<<<ceil_div(F + 1, 128), 128, 0, stream>>>(ukeys.p, nu, F, ustart.p);
    TGBM_CUDA(cudaStreamSynchronize(stream));
    k_feature_max_before<<<ceil_div(F + 1, 128), 128, 0, stream>>>(ukeys.p, ustart.p, before.p, nu, total, F, fmax.p, fbefore.p);
    std::vector<float> h_fmax(F);
    std::vector<long long> h_fbefore(F + 1);
    TGBM_CUDA(cudaMemcpyAsync(h_fmax.data(), fmax.p, sizeof(float) * F, cudaMemcpyDeviceToHost, stream));
    TGBM_CUDA(cudaMemcpyAsync(h_fbefore.data(), fbefore.p, sizeof(long long) * (F + 1), cudaMemcpyDeviceToHost, stream));
    TGBM_CUDA(cudaStreamSynchronize(stream));
    std::vector<ColumnShift> h_cs(F);
    std::vector<int> h_first(D), h_cols(D);
    std::vector<long long> h_sbefore(D);
    const int ave = F / D;
    for (int d = 0; d < D; ++d) {
        const int first = d * ave, ncol = d < D - 1 ? ave : F - first;
        h_first[d] = first; h_cols[d] = ncol; h_sbefore[d] = h_fbefore[first];
        float m = -INFINITY;
        for (int f = first; f < first + ncol; ++f) m = std::max(m, h_fmax[f]);
        // hist_cut.cu:109: the reference gives up when the shifted values leave the int range
        TGBM_CHECK(!(ncol > 0 && m > -INFINITY) || (double)m + (double)ncol * ((double)m + 1) < 2147483647.0,
                   "feature values too large for the column-sharded builder's value shift");
        for (int f = first; f < first + ncol; ++f)
            h_cs[f] = ColumnShift{d, first, m + 1.0f, h_fbefore[first + ncol] - h_fbefore[f + 1]};
    }
    DevBuf<ColumnShift> cs;
    DevBuf<int> shard_first, shard_cols;
    DevBuf<long long> shard_before;
    cs.alloc(F); shard_first.alloc(D); shard_cols.alloc(D); shard_before.alloc(D);
    TGBM_CUDA(cudaMemcpyAsync(cs.p, h_cs.data(), sizeof(ColumnShift) * F, cudaMemcpyHostToDevice, stream));
    TGBM_CUDA(cudaMemcpyAsync(shard_first.p, h_first.data(), sizeof(int) * D, cudaMemcpyHostToDevice, stream));
    TGBM_CUDA(cudaMemcpyAsync(shard_cols.p, h_cols.data(), sizeof(int) * D, cudaMemcpyHostToDevice, stream));
    TGBM_CUDA(cudaMemcpyAsync(shard_before.p, h_sbefore.data(), sizeof(long long) * D, cudaMemcpyHostToDevice, stream));
    // shift, sort per device (descending t), copies before every entry of the sorted array
    DevBuf<unsigned long long> k1, k2;
    DevBuf<long long> c2;
    k1.alloc(nu); k2.alloc(nu); c2.alloc(nu + 1);
    k_shift_keys<<<grid, 256, 0, stream>>>(ukeys.p, nu, cs.p, k1.p);
    {
        int end_bit = 32;
        while ((1ll << (end_bit - 32)) < D && end_bit < 64) ++end_bit;
        size_t tb = 0;
        cub::DeviceRadixSort::SortPairs(nullptr, tb, k1.p, k2.p, ucopies.p, c2.p, nu, 0, end_bit, stream);
        DevBuf<unsigned char> tmp;
        tmp.alloc(std::max<size_t>(tb, 1));
        cub::DeviceRadixSort::SortPairs(tmp.p, tb, k1.p, k2.p, ucopies.p, c2.p, nu, 0, end_bit, stream);
        TGBM_CUDA(cudaStreamSynchronize(stream));
    }
    scan(c2.p, before.p, nu);
    DevBuf<unsigned long long> n_heads;
    n_heads.alloc(1);
    n_heads.zero(stream);
    k_unshift_keys<<<grid, 256, 0, stream>>>(k2.p, before.p, nu, cs.p, shard_first.p, shard_cols.p, shard_before.p,
                                             k1.p, n_heads.p);
    unsigned long long h_heads = 0;
    TGBM_CUDA(cudaMemcpyAsync(&h_heads, n_heads.p, sizeof(h_heads), cudaMemcpyDeviceToHost, stream));
    {
        size_t tb = 0;
        cub::DeviceRadixSort::SortKeys(nullptr, tb, k1.p, k2.p, nu, 0, 64, stream);
        DevBuf<unsigned char> tmp;
        tmp.alloc(std::max<size_t>(tb, 1));
        cub::DeviceRadixSort::SortKeys(tmp.p, tb, k1.p, k2.p, nu, 0, 64, stream);
        TGBM_CUDA(cudaStreamSynchronize(stream));
    }
    nu = (long long)h_heads;
    ukeys.alloc(std::max<long long>(nu, 1));
    if (nu) TGBM_CUDA(cudaMemcpyAsync(ukeys.p, k2.p, sizeof(unsigned long long) * nu, cudaMemcpyDeviceToDevice, stream));
    TGBM_CUDA(cudaStreamSynchronize(stream));
}

// ------------------------------------------------------------------------------------------------
// Cut points (HistCut::get_cut_points_single, src/thundergbm/hist_cut.cu:205-286) and the bin matrix.
// Radix sort of (feature, value) keys and DeviceSelect::Unique come from CUB; this runs once, before
// the boosting loop.  With several ranks every rank contributes its sorted distinct keys, all ranks merge the lists and
// derive identical cut points from the union, so the bins equal the single-GPU ones.
void BoosterImpl::find_cuts_and_bins(const DataSet &ds) {
    const bool timing = getenv("TGBM_TIMING") != nullptr;  // phase times of the set-up on stderr
    auto t_prev = std::chrono::steady_clock::now();
    auto lap = [&](const char *what) {
        if (!timing) return;
        cudaStreamSynchronize(stream);
        const auto t = std::chrono::steady_clock::now();
        fprintf(stderr, "[tgbm init] %-28s %8.1f ms\n", what, std::chrono::duration<double, std::milli>(t - t_prev).count());
        t_prev = t;
    };
    const size_t nnz = (size_t)ds.rp[N];
    lap("H2D of the CSR");
    long long nu = 0;
    DevBuf<unsigned long long> ukeys;
    const bool multi = comm && comm->active();
    std::string local_err;  // see Booster::init: local phases are followed by an agreement of all ranks
    auto agree = [&](const char *what) {
        if (multi) comm->agree(local_err, what, stream);
        else if (!local_err.empty()) throw Error(local_err);
    };
    const bool colb = p.column_shards > 0;   // the column-sharded builder's cut points need the multiplicity of every key
    DevBuf<long long> ucopies;
    {
        DevBuf<unsigned long long> keys, keys2;
        DevBuf<long long> copies, copies2;
        DevBuf<long long> d_nu;
        DevBuf<long long> counts, mine;
        try {
            keys.alloc(std::max<size_t>(nnz, 1)); keys2.alloc(std::max<size_t>(nnz, 1)); d_nu.alloc(1);
            if (colb) { copies.alloc(std::max<size_t>(nnz, 1)); copies2.alloc(std::max<size_t>(nnz, 1)); }
            if (multi) { counts.alloc(comm->world); mine.alloc(1); }
        } catch (const std::exception &e) { local_err = e.what(); }
        auto sort_unique = [&](size_t n) -> long long {  // keys -> keys (sorted distinct), returns the count
            if (n == 0) return 0;
            size_t tb = 0;
            int end_bit = 32;
            while ((1ll << (end_bit - 32)) < F && end_bit < 64) ++end_bit;
            if (colb) {  // ... and copies -> copies (summed over equal keys)
                cub::DeviceRadixSort::SortPairs(nullptr, tb, keys.p, keys2.p, copies.p, copies2.p, (long long)n, 0, end_bit, stream);
                DevBuf<unsigned char> tmp;
                tmp.alloc(std::max<size_t>(tb, 16));
                cub::DeviceRadixSort::SortPairs(tmp.p, tb, keys.p, keys2.p, copies.p, copies2.p, (long long)n, 0, end_bit, stream);
                size_t tb2 = 0;
                cub::DeviceReduce::ReduceByKey(nullptr, tb2, keys2.p, keys.p, copies2.p, copies.p, d_nu.p, cub::Sum(), (long long)n, stream);
                DevBuf<unsigned char> tmp2;
                tmp2.alloc(std::max<size_t>(tb2, 16));
                cub::DeviceReduce::ReduceByKey(tmp2.p, tb2, keys2.p, keys.p, copies2.p, copies.p, d_nu.p, cub::Sum(), (long long)n, stream);
                long long r = 0;
                TGBM_CUDA(cudaMemcpyAsync(&r, d_nu.p, sizeof(long long), cudaMemcpyDeviceToHost, stream));
                TGBM_CUDA(cudaStreamSynchronize(stream));
                return r;
            }
            cub::DeviceRadixSort::SortKeys(nullptr, tb, keys.p, keys2.p, (long long)n, 0, end_bit, stream);
            DevBuf<unsigned char> tmp;
            tmp.alloc(std::max<size_t>(tb, 16));
            cub::DeviceRadixSort::SortKeys(tmp.p, tb, keys.p, keys2.p, (long long)n, 0, end_bit, stream);
            size_t tb2 = 0;
            cub::DeviceSelect::Unique(nullptr, tb2, keys2.p, keys.p, d_nu.p, (long long)n, stream);
            DevBuf<unsigned char> tmp2;
            tmp2.alloc(std::max<size_t>(tb2, 16));
            cub::DeviceSelect::Unique(tmp2.p, tb2, keys2.p, keys.p, d_nu.p, (long long)n, stream);
            long long r = 0;
            TGBM_CUDA(cudaMemcpyAsync(&r, d_nu.p, sizeof(long long), cudaMemcpyDeviceToHost, stream));
            TGBM_CUDA(cudaStreamSynchronize(stream));
            return r;
        };
        if (local_err.empty()) {
            try {
                if (nnz) k_make_keys<<<std::min(ceil_div(nnz, 256), num_sms * 16), 256, 0, stream>>>(d_val.p, d_col.p, nnz, keys.p);
                if (nnz && colb) k_fill_ll<<<std::min(ceil_div(nnz, 256), num_sms * 16), 256, 0, stream>>>(copies.p, nnz, 1);
                nu = sort_unique(nnz);
            } catch (const std::exception &e) { local_err = e.what(); }
        }
        agree("sorting its feature values");
        lap("  local sort + unique");
        if (multi) {
            // union of the ranks' distinct keys: all-gather (padded to the largest rank), then merge (or sort) + unique
            TGBM_CUDA(cudaMemcpyAsync(mine.p, &nu, sizeof(long long), cudaMemcpyHostToDevice, stream));
            comm->allgather(mine.p, counts.p, 1, Comm::I64, stream);
            std::vector<long long> hc(comm->world);
            TGBM_CUDA(cudaMemcpyAsync(hc.data(), counts.p, sizeof(long long) * comm->world, cudaMemcpyDeviceToHost, stream));
            comm->wait(stream);
            const long long mx = std::max<long long>(1, *std::max_element(hc.begin(), hc.end()));
            DevBuf<unsigned long long> padded, all;
            DevBuf<long long> padded_c, all_c;
            try {
                padded.alloc(mx); all.alloc((size_t)mx * comm->world);
                if (colb) { padded_c.alloc(mx); all_c.alloc((size_t)mx * comm->world); }
            } catch (const std::exception &e) { local_err = e.what(); }
            agree("making room for the ranks' feature values");
            TGBM_CUDA(cudaMemsetAsync(padded.p, 0xff, sizeof(unsigned long long) * mx, stream));
            if (nu) TGBM_CUDA(cudaMemcpyAsync(padded.p, keys.p, sizeof(unsigned long long) * nu, cudaMemcpyDeviceToDevice, stream));
            comm->allgather(padded.p, all.p, mx, Comm::I64, stream);
            lap("  all-gather of the distinct keys");
            if (colb) {
                TGBM_CUDA(cudaMemsetAsync(padded_c.p, 0, sizeof(long long) * mx, stream));
                if (nu) TGBM_CUDA(cudaMemcpyAsync(padded_c.p, copies.p, sizeof(long long) * nu, cudaMemcpyDeviceToDevice, stream));
                comm->allgather(padded_c.p, all_c.p, mx, Comm::I64, stream);
            }
            long long tot = 0;
            for (long long c : hc) tot += c;
            keys.alloc(std::max<long long>(tot, 1)); keys2.alloc(std::max<long long>(tot, 1));
            if (colb) { copies.alloc(std::max<long long>(tot, 1)); copies2.alloc(std::max<long long>(tot, 1)); }
            if (!colb && tot < INT_MAX) {
                // Every rank's list is sorted: the union is merged pairwise (log2 W passes over the keys) instead of
                // radix-sorted (five passes and a histogram), then made distinct.
                struct Run { const unsigned long long *p; long long n; };
                std::vector<Run> runs;
                for (int r = 0; r < comm->world; ++r)
                    if (hc[r]) runs.push_back({all.p + (size_t)r * mx, hc[r]});
                unsigned long long *bufs[2] = {keys.p, keys2.p};
                int into = 0;
                DevBuf<unsigned char> mtmp;
                while (runs.size() > 1) {
                    std::vector<Run> merged;
                    unsigned long long *out = bufs[into];
                    long long o = 0;
                    for (size_t i = 0; i + 1 < runs.size(); i += 2) {
                        size_t tb = 0;
                        cub::DeviceMerge::MergeKeys(nullptr, tb, runs[i].p, (int)runs[i].n, runs[i + 1].p, (int)runs[i + 1].n, out + o,
                                                    ::cuda::std::less<>{}, stream);
                        if (tb > mtmp.bytes() || !mtmp.p) mtmp.alloc(std::max<size_t>(tb, 16));
                        TGBM_CUDA(cub::DeviceMerge::MergeKeys(mtmp.p, tb, runs[i].p, (int)runs[i].n, runs[i + 1].p, (int)runs[i + 1].n, out + o,
                                                              ::cuda::std::less<>{}, stream));
                        merged.push_back({out + o, runs[i].n + runs[i + 1].n});
                        o += runs[i].n + runs[i + 1].n;
                    }
                    if (runs.size() & 1) {
                        const Run &last = runs.back();
                        TGBM_CUDA(cudaMemcpyAsync(out + o, last.p, sizeof(unsigned long long) * last.n, cudaMemcpyDeviceToDevice, stream));
                        merged.push_back({out + o, last.n});
                    }
                    runs.swap(merged);
                    into ^= 1;
                }
                nu = 0;
                if (!runs.empty()) {
                    size_t tb = 0;
                    cub::DeviceSelect::Unique(nullptr, tb, runs[0].p, bufs[into], d_nu.p, runs[0].n, stream);
                    DevBuf<unsigned char> tmp;
                    tmp.alloc(std::max<size_t>(tb, 16));
                    TGBM_CUDA(cub::DeviceSelect::Unique(tmp.p, tb, runs[0].p, bufs[into], d_nu.p, runs[0].n, stream));
                    TGBM_CUDA(cudaMemcpyAsync(&nu, d_nu.p, sizeof(long long), cudaMemcpyDeviceToHost, stream));
                    TGBM_CUDA(cudaStreamSynchronize(stream));
                    if (into == 1) std::swap(keys.p, keys2.p);   // the distinct keys are expected in `keys`
                }
            } else {
                long long o = 0;
                for (int r = 0; r < comm->world; ++r) {
                    if (hc[r]) TGBM_CUDA(cudaMemcpyAsync(keys.p + o, all.p + (size_t)r * mx, sizeof(unsigned long long) * hc[r], cudaMemcpyDeviceToDevice, stream));
                    if (hc[r] && colb) TGBM_CUDA(cudaMemcpyAsync(copies.p + o, all_c.p + (size_t)r * mx, sizeof(long long) * hc[r], cudaMemcpyDeviceToDevice, stream));
                    o += hc[r];
                }
                nu = sort_unique(tot);
            }
            lap("  union of the ranks' keys");
        }
        ukeys.alloc(std::max<long long>(nu, 1));
        if (nu) TGBM_CUDA(cudaMemcpyAsync(ukeys.p, keys.p, sizeof(unsigned long long) * nu, cudaMemcpyDeviceToDevice, stream));
        if (colb) {
            ucopies.alloc(std::max<long long>(nu, 1) + 1);
            if (nu) TGBM_CUDA(cudaMemcpyAsync(ucopies.p, copies.p, sizeof(long long) * nu, cudaMemcpyDeviceToDevice, stream));
        }
        TGBM_CUDA(cudaStreamSynchronize(stream));
    }
    if (colb) column_builder_candidates(ukeys, ucopies, nu);
    lap("sort + unique of the keys");
    // distinct values per feature -> stride and number of cut points per feature (host, F+1 numbers)
    DevBuf<long long> ustart;
    ustart.alloc(F + 1);
    k_feature_bounds<<<ceil_div(F + 1, 128), 128, 0, stream>>>(ukeys.p, nu, F, ustart.p);
    std::vector<long long> h_ustart(F + 1);
    TGBM_CUDA(cudaMemcpyAsync(h_ustart.data(), ustart.p, sizeof(long long) * (F + 1), cudaMemcpyDeviceToHost, stream));
    TGBM_CUDA(cudaStreamSynchronize(stream));
    std::vector<int> h_stride(F);
    h_cut_ptr.assign(F + 1, 0);
    for (int f = 0; f < F; ++f) {
        const long long u = h_ustart[f + 1] - h_ustart[f];
        const long long s = u / p.max_num_bin;
        h_stride[f] = (int)s;
        h_cut_ptr[f + 1] = h_cut_ptr[f] + (int)(s == 0 ? u : p.max_num_bin);
    }
    B = h_cut_ptr[F];
    DevBuf<int> d_stride;
    d_stride.alloc(std::max(F, 1));
    cut_ptr.alloc(F + 1); cut_val.alloc(std::max(B, 1)); cut_fid.alloc(std::max(B, 1));
    TGBM_CUDA(cudaMemcpyAsync(d_stride.p, h_stride.data(), sizeof(int) * F, cudaMemcpyHostToDevice, stream));
    TGBM_CUDA(cudaMemcpyAsync(cut_ptr.p, h_cut_ptr.data(), sizeof(int) * (F + 1), cudaMemcpyHostToDevice, stream));
    if (nu) k_select_cuts<<<std::min(ceil_div(nu, 256), num_sms * 16), 256, 0, stream>>>(ukeys.p, nu, ustart.p, d_stride.p, cut_ptr.p,
                                                                                         p.max_num_bin, cut_val.p, cut_fid.p, colb ? 1 : 0);
    h_cut_val.resize(B);
    TGBM_CUDA(cudaMemcpyAsync(h_cut_val.data(), cut_val.p, sizeof(float) * B, cudaMemcpyDeviceToHost, stream));

    lap("cut point selection");
    // Layout: dense byte matrices (row-major + column-major) unless they would dwarf the data itself -- then the
    // reference's CSR of global bin ids.  TGBM_LAYOUT=dense|sparse overrides the choice (tests).
    {
        const double dense_bytes = 2.0 * (double)N * Fpad, csr_bytes = 4.0 * (double)nnz;
        sparse = F > 256 && dense_bytes > 4.0 * csr_bytes;
        if (const char *e = getenv("TGBM_LAYOUT")) {
            if (!strcmp(e, "sparse")) sparse = true;
            if (!strcmp(e, "dense")) sparse = false;
        }
        TGBM_CHECK(sparse || (long long)F * 32 <= (1 << 21), "the dense bin matrix supports at most 65536 features");
    }
    nnz_local = (long long)nnz;
    if (sparse) {
        sp_row_ptr.alloc(N + 1);
        sp_bin.alloc(std::max<size_t>(nnz, 1));
        TGBM_CUDA(cudaMemcpyAsync(sp_row_ptr.p, d_row_ptr.p, sizeof(int) * (N + 1), cudaMemcpyDeviceToDevice, stream));
        if (nnz) k_bin_csr<<<std::min(ceil_div(nnz, 256), num_sms * 16), 256, 0, stream>>>(d_col.p, d_val.p, nnz, cut_ptr.p, cut_val.p, sp_bin.p, colb ? 1 : 0);
        // rows whose columns arrive unordered are put in ascending bin order (= ascending column order)
        if (nnz) {
            DevBuf<int> unsorted;
            unsorted.alloc(1);
            TGBM_CUDA(cudaMemsetAsync(unsorted.p, 0, sizeof(int), stream));
            k_rows_unsorted<<<std::min(ceil_div(N, 256), num_sms * 16), 256, 0, stream>>>(sp_row_ptr.p, sp_bin.p, N, unsorted.p);
            int h_unsorted = 0;
            TGBM_CUDA(cudaMemcpyAsync(&h_unsorted, unsorted.p, sizeof(int), cudaMemcpyDeviceToHost, stream));
            TGBM_CUDA(cudaStreamSynchronize(stream));
            if (h_unsorted) {
                DevBuf<int> sorted_bin;
                sorted_bin.alloc(nnz);
                size_t tmp_bytes = 0;
                TGBM_CUDA(cub::DeviceSegmentedSort::SortKeys(nullptr, tmp_bytes, sp_bin.p, sorted_bin.p, (long long)nnz, (long long)N, sp_row_ptr.p,
                                                             sp_row_ptr.p + 1, stream));
                DevBuf<unsigned char> tmp;
                tmp.alloc(std::max<size_t>(tmp_bytes, 1));
                TGBM_CUDA(cub::DeviceSegmentedSort::SortKeys(tmp.p, tmp_bytes, sp_bin.p, sorted_bin.p, (long long)nnz, (long long)N, sp_row_ptr.p,
                                                             sp_row_ptr.p + 1, stream));
                TGBM_CUDA(cudaMemcpyAsync(sp_bin.p, sorted_bin.p, sizeof(int) * nnz, cudaMemcpyDeviceToDevice, stream));
                TGBM_CUDA(cudaStreamSynchronize(stream));
            }
        }
        // chunks of whole features with at most 256 bins for the split evaluation
        std::vector<int> cb(1, 0);
        int cur = 0;
        for (int f = 0; f < F; ++f) {
            const int nbf = h_cut_ptr[f + 1] - h_cut_ptr[f];
            if (cur + nbf > 256 && cur > 0) { cb.push_back(h_cut_ptr[f]); cur = 0; }
            cur += nbf;
        }
        if (cb.back() != B) cb.push_back(B);
        n_chunks = (int)cb.size() - 1;
        chunk_bin0.alloc(cb.size());
        TGBM_CUDA(cudaMemcpyAsync(chunk_bin0.p, cb.data(), sizeof(int) * cb.size(), cudaMemcpyHostToDevice, stream));
        TGBM_CUDA(cudaStreamSynchronize(stream));
    } else {
        bins.alloc((size_t)N * Fpad);
        binsT.alloc((size_t)F * Npad);
        TGBM_CUDA(cudaMemsetAsync(bins.p, MISSING_BIN, bins.bytes(), stream));
        TGBM_CUDA(cudaMemsetAsync(binsT.p, MISSING_BIN, binsT.bytes(), stream));
        if (N) k_bin_dense<<<ceil_div(N, 128), 128, 0, stream>>>(d_row_ptr.p, d_col.p, d_val.p, N, cut_ptr.p, cut_val.p, Fpad, Npad, bins.p, binsT.p, colb ? 1 : 0);
    }
    TGBM_CUDA(cudaStreamSynchronize(stream));
    TGBM_CUDA(cudaGetLastError());
    d_row_ptr.release(); d_col.release(); d_val.release();
    lap("binning");
}

// ------------------------------------------------------------------------------------------------
// Exact builder, set-up: the stored values by column, largest first (SparseColumns::csr2csc_gpu,
// src/thundergbm/sparse_columns.cu:20-93 and :127) -- one stable radix sort of (column, complement of the value's ordered
// image) keys with the row ids as payload -- and the buffers of the level loop, sized once.
void BoosterImpl::init_exact(const DataSet &ds) {
    const size_t nnz = (size_t)ds.rp[N];
    ex_nnz = (long long)nnz;
    TGBM_CHECK(nnz < (1ull << 31), "the exact builder indexes stored values with 32 bits");
    TGBM_CHECK((double)F * (double)(1 << std::max(0, depth - 1)) < 4294967295.0, "columns x nodes of the last level must fit 32 bits");
    const size_t n1 = std::max<size_t>(nnz, 1);
    const int grid = std::max(1, std::min(ceil_div((long long)n1, 256), num_sms * 16));
    {
        DevBuf<unsigned long long> keys, keys2;
        DevBuf<int> rows;
        keys.alloc(n1); keys2.alloc(n1); rows.alloc(n1); ex_row.alloc(n1); ex_val.alloc(n1); ex_csc_ptr.alloc(F + 1);
        if (N) k_exact_rows<<<std::min(ceil_div(N, 256), num_sms * 16), 256, 0, stream>>>(d_row_ptr.p, N, rows.p);
        if (nnz) k_exact_csc_keys<<<grid, 256, 0, stream>>>(d_val.p, d_col.p, nnz, keys.p);
        int end_bit = 32;
        while ((1ll << (end_bit - 32)) < F && end_bit < 64) ++end_bit;
        if (nnz) {
            size_t tb = 0;
            cub::DeviceRadixSort::SortPairs(nullptr, tb, keys.p, keys2.p, rows.p, ex_row.p, (long long)nnz, 0, end_bit, stream);
            DevBuf<unsigned char> tmp;
            tmp.alloc(std::max<size_t>(tb, 1));
            TGBM_CUDA(cub::DeviceRadixSort::SortPairs(tmp.p, tb, keys.p, keys2.p, rows.p, ex_row.p, (long long)nnz, 0, end_bit, stream));
            k_exact_csc_vals<<<grid, 256, 0, stream>>>(keys2.p, nnz, ex_val.p);
            TGBM_CUDA(cudaStreamSynchronize(stream));
        }
        k_feature_bounds<<<ceil_div(F + 1, 128), 128, 0, stream>>>(keys2.p, (long long)nnz, F, ex_csc_ptr.p);
        TGBM_CUDA(cudaStreamSynchronize(stream));
    }
    d_row_ptr.release(); d_col.release(); d_val.release();
    // no cut points, no bin matrix
    B = 0; sparse = false;
    h_cut_ptr.assign(F + 1, 0);
    cut_ptr.alloc(F + 1); cut_val.alloc(1); cut_fid.alloc(1);
    cut_ptr.zero(stream);
    const size_t max_nl = (size_t)1 << std::max(0, depth - 1);
    for (int i = 0; i < 2; ++i) { ex_key[i].alloc(n1); ex_idx[i].alloc(n1); }
    k_exact_iota<<<grid, 256, 0, stream>>>(ex_idx[0].p, n1);
    ex_sums.alloc(n1 * (f32 ? sizeof(ExPair<float>) : sizeof(ExPair<long long>)));
    ex_pid_ptr.alloc((size_t)F * max_nl + 2);
    ex_nid.alloc(std::max(N, 1));
    ex_best.alloc(max_nl);
    ex_best.zero(stream);
    ex_any.alloc(1);
    ex_any.zero(stream);
    size_t tb_sort = 0, tb_scan = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, tb_sort, ex_key[0].p, ex_key[1].p, ex_idx[0].p, ex_idx[1].p, (long long)n1, 0, 32, stream);
    if (f32) {
        cub::TransformInputIterator<ExPair<float>, ExGather<float>, cub::CountingInputIterator<long long>> in(
            cub::CountingInputIterator<long long>(0), ExGather<float>{ex_idx[1].p, ex_row.p, nullptr});
        cub::DeviceScan::InclusiveScanByKey(nullptr, tb_scan, ex_key[1].p, in, reinterpret_cast<ExPair<float> *>(ex_sums.p), ExAdd<float>(),
                                            (long long)n1, cub::Equality(), stream);
    } else {
        cub::TransformInputIterator<ExPair<long long>, ExGather<long long>, cub::CountingInputIterator<long long>> in(
            cub::CountingInputIterator<long long>(0), ExGather<long long>{ex_idx[1].p, ex_row.p, nullptr});
        cub::DeviceScan::InclusiveScanByKey(nullptr, tb_scan, ex_key[1].p, in, reinterpret_cast<ExPair<long long> *>(ex_sums.p), ExAdd<long long>(),
                                            (long long)n1, cub::Equality(), stream);
    }
    ex_tmp.alloc(std::max<size_t>(std::max(tb_sort, tb_scan), 1));
    TGBM_CUDA(cudaFuncSetAttribute(k_exact_gain<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    TGBM_CUDA(cudaFuncSetAttribute(k_exact_gain<long long>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    TGBM_CUDA(cudaStreamSynchronize(stream));
    TGBM_CUDA(cudaGetLastError());
}

// The level loop of one tree with the exact split search (TreeBuilder::build_approximate, tree_builder.cu:147-194, with
// ExactTreeBuilder::find_split / update_ins2node_id).  T = float: the reference's arithmetic; T = long long: sums of the
// quantised gradients, exact in any order.
template <typename T>
void BoosterImpl::exact_levels(int k, const void *gh_rows) {
    const long long nnz = ex_nnz;
    const int grid = std::max(1, std::min(ceil_div(std::max<long long>(nnz, 1), 256), num_sms * 16));
    const int row_grid = std::max(1, std::min(ceil_div(std::max(N, 1), 256), num_sms * 8));
    ExPair<T> *sums = reinterpret_cast<ExPair<T> *>(ex_sums.p);
    TGBM_CUDA(cudaMemsetAsync(ex_nid.p, 0, sizeof(int) * (size_t)std::max(N, 1), stream));
    for (int level = 0; level < depth; ++level) {
        const int nl = 1 << level;
        const long long n_pid = (long long)F * nl;
        if (nnz) {
            k_exact_keys<<<grid, 256, 0, stream>>>(ex_row.p, nnz, ex_csc_ptr.p, F, ex_nid.p, level, ex_key[0].p);
            int end_bit = 1;
            while ((1ll << end_bit) <= n_pid && end_bit < 32) ++end_bit;   // the largest key, EX_NONE, has every bit set
            size_t tb = ex_tmp.n;
            TGBM_CUDA(cub::DeviceRadixSort::SortPairs(ex_tmp.p, tb, ex_key[0].p, ex_key[1].p, ex_idx[0].p, ex_idx[1].p, nnz, 0, end_bit, stream));
            using Gather = ExGather<T>;
            cub::TransformInputIterator<ExPair<T>, Gather, cub::CountingInputIterator<long long>> in(
                cub::CountingInputIterator<long long>(0),
                Gather{ex_idx[1].p, ex_row.p, reinterpret_cast<decltype(Gather::gh)>(gh_rows)});
            tb = ex_tmp.n;
            TGBM_CUDA(cub::DeviceScan::InclusiveScanByKey(ex_tmp.p, tb, ex_key[1].p, in, sums, ExAdd<T>(), nnz, cub::Equality(), stream));
            k_exact_pid_ptr<<<std::max(1, std::min(ceil_div(n_pid + 1, 256), num_sms * 16)), 256, 0, stream>>>(ex_key[1].p, nnz, n_pid, ex_pid_ptr.p);
            k_exact_gain<T><<<num_sms * 2, EX_THREADS, sizeof(unsigned long long) * (size_t)nl, stream>>>(
                ex_key[1].p, ex_idx[1].p, ex_val.p, sums, ex_pid_ptr.p, nnz, level, nodes.p, qinfo.p, p.min_child_weight, p.lambda,
                ignored_all.p, rstate.p, F, ex_best.p);
            launches += 5;
        }
        k_exact_apply<T><<<ceil_div(nl, 128), 128, 0, stream>>>(ex_key[1].p, ex_idx[1].p, ex_val.p, sums, ex_pid_ptr.p, level, nodes.p, qinfo.p,
                                                                 p.min_child_weight, p.lambda, p.rt_eps, ex_best.p, ex_any.p);
        if (nnz) k_exact_move<<<grid, 256, 0, stream>>>(ex_row.p, ex_val.p, nnz, ex_csc_ptr.p, F, ex_nid.p, nodes.p, ex_any.p);
        k_exact_move_missing<<<row_grid, 256, 0, stream>>>(ex_nid.p, N, level, nodes.p, ex_any.p);
        launches += 3;
    }
    (void)k;
}

void BoosterImpl::build_tree_exact(int round, int k) {
    const int tree_index = round * K + k;
    k_tree_init<<<ceil_div(n_nodes, 256), 256, 0, stream>>>(nodes.p, n_nodes, root_sum.p + 2 * k, qinfo.p, p.lambda, N,
                                                            seg_begin[0].p, seg_cnt[0].p, gcnt.p, ctl.p, f32 ? 1 : 0);
    if (f32) exact_levels<float>(k, gh.p + (size_t)k * N);
    else exact_levels<long long>(k, ghq.p + (size_t)k * N);
    k_prune<<<1, 1024, prune_in_smem ? sizeof(TreeNode) * (size_t)n_nodes : 0, stream>>>(nodes.p, n_nodes, depth, p.gamma, prune_in_smem ? 1 : 0);
    if (N) {
        int *nid_out = p.keep_nid ? nid_keep.p + (size_t)tree_index * N : nullptr;
        k_exact_predict<<<std::min(ceil_div(N, 256), num_sms * 8), 256, 0, stream>>>(ex_nid.p, N, nodes.p, p.learning_rate, ypred.p + (size_t)k * N, nid_out);
    }
    grad_max_ready = metric_partial_ready = false;
    k_store_tree<<<std::min(ceil_div(n_nodes, 256), 64), 256, 0, stream>>>(nodes.p, model.p, n_nodes, K, k, rstate.p);
    launches += 4;
}

// ------------------------------------------------------------------------------------------------
Booster::Booster(const GBMParam &param, const Comm *comm) : impl_(new BoosterImpl) {
    impl_->p = param;
    impl_->comm = comm;
}
Booster::~Booster() = default;

void Booster::init(const DataSet &ds) {
    BoosterImpl &m = *impl_;
    GBMParam &p = m.p;
    m.objective = objective_from_name(p.objective);
    TGBM_CHECK(m.objective != OBJ_UNKNOWN, "undefined objective " + p.objective);
    TGBM_CHECK(p.depth >= 1 && p.depth <= 14, "depth must be in [1, 14]");
    TGBM_CHECK(p.max_num_bin >= 1 && p.max_num_bin <= 255, "max_num_bin must be in [1, 255] (bin ids are bytes, 255 marks a missing value)");
    TGBM_CHECK(p.quant_bits >= 8 && p.quant_bits <= 20, "quant_bits must be in [8, 20]");
    TGBM_CHECK(p.hist_mode == 0 || p.hist_mode == 1, "hist_mode must be 0 (fp32) or 1 (exact)");
    m.f32 = p.hist_mode == 0;
    TGBM_CHECK(p.column_sampling_rate > 0.f, "column_sampling_rate must be positive");
    int dev = 0;
    TGBM_CUDA(cudaGetDevice(&dev));
    TGBM_CUDA(cudaDeviceGetAttribute(&m.num_sms, cudaDevAttrMultiProcessorCount, dev));
    TGBM_CUDA(cudaStreamCreateWithFlags(&m.stream, cudaStreamNonBlocking));
    TGBM_CUDA(cudaStreamCreateWithFlags(&m.stream2, cudaStreamNonBlocking));
    TGBM_CUDA(cudaEventCreateWithFlags(&m.ev_scan, cudaEventDisableTiming));
    TGBM_CUDA(cudaEventCreateWithFlags(&m.ev_plan, cudaEventDisableTiming));
    m.N = ds.n_rows;
    m.F = ds.n_features;
    m.depth = p.depth;
    m.n_nodes = (1 << (p.depth + 1)) - 1;
    m.label = ds.label;
    const bool multi = m.comm && m.comm->active();
    // Every phase that can fail on one rank alone (a check of this rank's input, an allocation) runs under `locally`
    // and is followed by an agreement of all ranks, so that no rank enters a collective its peers will never join.
    std::string local_err;
    auto locally = [&](auto &&phase) {
        try { phase(); } catch (const std::exception &e) { local_err = e.what(); }
    };
    auto agree = [&](const char *what) {
        if (multi) m.comm->agree(local_err, what, m.stream);
        else if (!local_err.empty()) throw Error(local_err);
    };
    // (buffers of the collectives are allocated inside the local phases too: between an agreement and the launch of the
    // collective no rank makes a call that could wait for another device -- cudaMalloc can, once peer access is on)
    DevBuf<long long> mine, all;
    locally([&] {
        if (need_group_file(m.objective)) RankState::validate(ds, m.N);
        m.upload_csr(ds);
        if (multi) { mine.alloc(3); all.alloc(3 * (size_t)m.comm->world); }
    });
    agree("loading its rows");

    // global row count, this rank's row offset, global feature count, query groups before this rank's
    m.N_global = m.N;
    m.row_offset = 0;
    long long first_group = 0, total_groups = (long long)ds.group.size();
    if (multi) {
        long long h[3] = {m.N, m.F, (long long)ds.group.size()};
        TGBM_CUDA(cudaMemcpyAsync(mine.p, h, sizeof(h), cudaMemcpyHostToDevice, m.stream));
        m.comm->allgather(mine.p, all.p, 3, Comm::I64, m.stream);
        std::vector<long long> ha(3 * (size_t)m.comm->world);
        TGBM_CUDA(cudaMemcpyAsync(ha.data(), all.p, sizeof(long long) * ha.size(), cudaMemcpyDeviceToHost, m.stream));
        m.comm->wait(m.stream);
        m.N_global = 0;
        total_groups = 0;
        for (int r = 0; r < m.comm->world; ++r) {
            if (r < m.comm->rank) { m.row_offset += ha[3 * r]; first_group += ha[3 * r + 2]; }
            m.N_global += ha[3 * r];
            m.F = std::max<int>(m.F, (int)ha[3 * r + 1]);
            total_groups += ha[3 * r + 2];
        }
    }
    TGBM_CHECK(m.N_global < (1ll << 31), "row count must fit 32 bits");
    TGBM_CHECK(m.F >= 1, "data set has no features");
    m.Fpad = (m.F + 31) / 32 * 32;
    m.G = m.Fpad / 32;
    m.Npad = ((size_t)m.N + 127) / 128 * 128;

    // number of classes / trees per round (src/thundergbm/trainer.cu:26-37)
    m.K = 1;
    if (need_group_label(m.objective)) {
        p.num_class = (int)ds.label.size();
        if (p.num_class > 2) m.K = p.num_class;
    } else if (m.objective == REG_LINEAR || m.objective == REG_LOGISTIC) {
        p.num_class = 1;
    }
    p.tree_per_rounds = m.K;
    // with two labels the reference's Softmax::get_gradient aborts on a size check (multiclass_obj.cu:9); binary:logistic is the 2-class objective
    TGBM_CHECK(!((m.objective == MULTI_SOFTMAX || m.objective == MULTI_SOFTPROB) && p.num_class <= 2),
               "multi:softmax / multi:softprob need more than two classes; use binary:logistic for two");
    m.num_class = p.num_class;

    const bool timing = getenv("TGBM_TIMING") != nullptr;
    auto t_mark = std::chrono::steady_clock::now();
    auto lap = [&](const char *what) {
        if (!timing) return;
        cudaStreamSynchronize(m.stream);
        const auto t = std::chrono::steady_clock::now();
        fprintf(stderr, "[tgbm init] %-28s %8.1f ms\n", what, std::chrono::duration<double, std::milli>(t - t_mark).count());
        t_mark = t;
    };
    if (p.tree_method == "auto") p.tree_method = m.F > 20000 ? "exact" : "hist";   // src/thundergbm/trainer.cu:19-23
    TGBM_CHECK(p.tree_method == "hist" || p.tree_method == "exact", "unknown tree_method " + p.tree_method);
    m.exact = p.tree_method == "exact";
    if (m.exact) {
        TGBM_CHECK(!multi, "the exact builder runs on one GPU");
        locally([&] { m.init_exact(ds); });
        agree("sorting its columns");
    } else {
        m.find_cuts_and_bins(ds);
    }
    lap("= cuts and bins, with frees");

    locally([&] {
    const int N = m.N, K = m.K, depth = m.depth;
    const size_t n1 = std::max<size_t>(N, 1);
    m.y.alloc(n1); m.ypred.alloc(n1 * K); m.gh.alloc(n1 * K); m.ghq.alloc(n1 * K);
    upload_h2d(m.y.p, ds.yv ? ds.yv : ds.y.data(), sizeof(float) * (size_t)N, m.stream, std::min(4, upload_threads()));
    if (ds.labels_raw && N) {  // label value -> class index (dataset.cpp:83-101), on the device
        DevBuf<float> d_label;
        d_label.alloc(std::max<size_t>(ds.label.size(), 1));
        TGBM_CUDA(cudaMemcpyAsync(d_label.p, ds.label.data(), sizeof(float) * ds.label.size(), cudaMemcpyHostToDevice, m.stream));
        k_map_labels<<<std::min(ceil_div(N, 256), m.num_sms * 8), 256, 0, m.stream>>>(m.y.p, N, d_label.p, (int)ds.label.size());
        TGBM_CUDA(cudaStreamSynchronize(m.stream));
    }
    m.ypred.zero(m.stream);
    m.maxbits.alloc(2); m.root_sum.alloc(2 * (size_t)K); m.qinfo.alloc(1);
    if (p.bagging) {
        TGBM_CHECK((unsigned long long)std::max(p.num_class, 1) * (unsigned long long)m.N_global < (1ull << 32), "bagging: num_class x rows must fit 32 bits");
        m.bag_count.alloc(n1 * K);
    }
    if (p.column_sampling_rate < 1.f) {
        // Shard::column_sampling (src/thundergbm/builder/shard.cu:8-23), once per round for all trees of the round:
        // max(1, int(F * rate)) randomly chosen features are put into the IGNORED set -- the reference's rate is the
        // share that is left out.  Its shuffle draws from std::rand(); here the features with the smallest hash of
        // (seed, round, feature) are taken, for all rounds in advance (the boosting loop never returns to the host).
        const int F = m.F, rounds = std::max(p.n_trees, 1);
        const int n_ignored = std::max(1, (int)(F * p.column_sampling_rate));
        std::vector<unsigned char> mask((size_t)rounds * F, 0);
        std::vector<std::pair<uint32_t, int>> key(F);
        for (int r = 0; r < rounds; ++r) {
            for (int f = 0; f < F; ++f) key[f] = {mix32(p.sample_seed ^ 0xC01A5EEDu, (uint32_t)r, 0u, (uint32_t)f), f};
            std::nth_element(key.begin(), key.begin() + std::min(n_ignored, F) - 1, key.end());
            for (int i = 0; i < std::min(n_ignored, F); ++i) mask[(size_t)r * F + key[i].second] = 1;
        }
        m.ignored_all.alloc(mask.size());
        TGBM_CUDA(cudaMemcpyAsync(m.ignored_all.p, mask.data(), mask.size(), cudaMemcpyHostToDevice, m.stream));
        TGBM_CUDA(cudaStreamSynchronize(m.stream));
    }
    m.qinfo_log.alloc(std::max(p.n_trees, 1) + 1);
    m.nodes.alloc(m.n_nodes);
    m.model.alloc((size_t)std::max(p.n_trees, 1) * K * m.n_nodes);
    m.metric.alloc(std::max(p.n_trees, 1));
    for (int i = 0; i < 2; ++i) {
        // left children in the first half, right children in the second (single-pass partition); the bulk copies that
        // stage a unit of records read up to a unit beyond the last record
        m.rec_idx[i].alloc(2 * n1 + 2 * F32_THREADS); m.rec_gh[i].alloc(2 * n1 + 2 * F32_THREADS);
        m.seg_begin[i].alloc((size_t)1 << depth); m.seg_cnt[i].alloc((size_t)1 << depth);
        m.seg_begin[i].zero(m.stream); m.seg_cnt[i].zero(m.stream);
    }
    m.gcnt.alloc((size_t)1 << depth);
    m.gcnt.zero(m.stream);
    if (p.keep_nid) m.nid_keep.alloc(n1 * K * std::max(p.n_trees, 1));
    const size_t B1 = std::max(m.B, 1);
    m.hist_full.alloc((((size_t)1 << depth) - 1) * B1 * 2);
    m.hist_built.alloc(std::max<size_t>(1, (size_t)1 << std::max(0, depth - 2)) * B1 * 2);
    const int max_pairs = std::max(1, 1 << std::max(0, depth - 2));
    if (m.f32) {
        for (int f = 0; f < std::min(m.F, 256); ++f) m.f32_cuts.v[f] = m.h_cut_ptr[f];
        m.spread_cells = std::max<size_t>(std::min<size_t>((size_t)32 * max_pairs * B1, (size_t)8 << 20), (size_t)max_pairs * B1);  // <= 64 MB
        m.hist_spread.alloc(m.spread_cells);
        m.sum_partial.alloc((size_t)SUM_BLOCKS * K * 2);
        const QuantInfo one{1.0, 1.0, 1.0, 1.0};
        TGBM_CUDA(cudaMemcpyAsync(m.qinfo.p, &one, sizeof(one), cudaMemcpyHostToDevice, m.stream));
        TGBM_CUDA(cudaStreamSynchronize(m.stream));
    }
    m.built_right.alloc(max_pairs); m.hist_work.alloc(max_pairs); m.hist_tile_base.alloc(max_pairs + 1);
    m.hist_cta_off.alloc((size_t)m.num_sms + 1);
    m.eval_ticket.alloc(max_pairs);
    m.rstate.alloc(1);
    m.rstate.zero(m.stream);
    m.graphs_allowed = getenv("TGBM_NO_GRAPH") == nullptr;
    m.eval_ticket.zero(m.stream);
    m.hist_seq.alloc((size_t)ceil_div(std::max(N, 1), HIST_THREADS) + max_pairs + 16);
    m.recs.alloc(m.exact ? 1 : ((size_t)1 << (depth - 1)) * (m.sparse ? std::max(m.n_chunks, 1) : m.F));
    m.max_tiles = ceil_div(N, PART_TILE) + (1 << depth) + 2;
    m.tile_left.alloc(m.max_tiles);
    m.tile_node[0].alloc(m.max_tiles); m.tile_node[1].alloc(m.max_tiles);
    m.node_tile0[0].alloc(((size_t)1 << depth) + 1); m.node_tile0[1].alloc(((size_t)1 << depth) + 1);
    m.bits.alloc((size_t)m.max_tiles * (PART_TILE / 32));
    m.part_base.alloc((size_t)1 << depth);
    m.part_status.alloc(m.max_tiles);
    m.part_status.zero(m.stream);
    m.part_group.alloc(m.max_tiles / 32 + 2);
    m.part_group.zero(m.stream);
    m.part_one = getenv("TGBM_PART_ONE") != nullptr;
    m.f32_staged = getenv("TGBM_NO_BULK_COPY") == nullptr;
    m.ctl.alloc(1);
    m.ctl.zero(m.stream);
    m.metric_partial.alloc(1024); m.metric_sum.alloc(1);
    m.window_rows = (1 << (31 - p.quant_bits)) - HIST_THREADS;
    TGBM_CHECK(m.window_rows >= HIST_THREADS, "quant_bits too large for the int32 accumulation window");
    m.hist_smem = 2 * 256 * 32 * 4 + 2 * 256 * 32 * 8;  // int32 accumulators + int64 totals, both [2][256 bins][32 features]
    TGBM_CUDA(cudaFuncSetAttribute(k_hist<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, m.hist_smem));
    TGBM_CUDA(cudaFuncSetAttribute(k_hist<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, m.hist_smem));
    TGBM_CUDA(cudaFuncSetAttribute(k_predict_walk<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TGBM_CUDA(cudaFuncSetAttribute(k_predict_walk<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TGBM_CUDA(cudaFuncSetAttribute(k_predict_walk<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TGBM_CUDA(cudaFuncSetAttribute(k_hist_sparse<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SPARSE_SMEM_BINS * 16));
    TGBM_CUDA(cudaFuncSetAttribute(k_hist_sparse<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SPARSE_SMEM_BINS * 16));
    m.prune_in_smem = sizeof(TreeNode) * (size_t)m.n_nodes <= 200 * 1024;  // up to depth 11
    if (m.prune_in_smem && sizeof(TreeNode) * (size_t)m.n_nodes > 48 * 1024)
        TGBM_CUDA(cudaFuncSetAttribute(k_prune, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(TreeNode) * (size_t)m.n_nodes)));
    if (need_group_file(m.objective)) m.rank.init(ds, m.objective, m.N, m.stream, first_group, total_groups);
    });
    agree("allocating its training buffers");
    lap("training buffers");
    m.init_base_score();
    TGBM_CUDA(cudaStreamSynchronize(m.stream));
    TGBM_CUDA(cudaGetLastError());
    lap("base score");
}

// ------------------------------------------------------------------------------------------------
void BoosterImpl::gradient(int round) {
    const int tb = 256;
    const bool pointwise = objective == REG_LINEAR || objective == REG_LOGISTIC || objective == BINARY_LOGISTIC;
    const int logistic = objective == REG_LINEAR ? 0 : 1;
    // the pass that applied the previous tree has already found this round's gradient maxima
    const bool have_max = pointwise && grad_max_ready && round >= 0 && !f32 && !p.bagging;
    grad_max_ready = false;
    root_sum.zero(stream);
    if (!have_max) {
        maxbits.zero(stream);
        if (N) {
            const int gb = std::max(1, std::min(ceil_div(N, tb), num_sms * 8));
            switch (objective) {
            case REG_LINEAR: case REG_LOGISTIC: case BINARY_LOGISTIC:
                k_grad_pointwise<<<gb, tb, 0, stream>>>(y.p, ypred.p, N, logistic, gh.p, maxbits.p); break;
            case MULTI_SOFTMAX: case MULTI_SOFTPROB:
                k_grad_softmax<<<gb, tb, 0, stream>>>(y.p, ypred.p, N, K, gh.p, maxbits.p); break;
            case RANK_PAIRWISE: case RANK_NDCG:
                rank.gradient(rstate.p, p.rank_seed, ypred.p, gh.p, maxbits.p, stream); break;
            }
            ++launches;
        }
    }
    if (p.bagging && round >= 0 && N) {  // not for the base score (include/thundergbm/booster.h:69-73 comes before any sampling)
        bag_count.zero(stream);
        const unsigned long long m_total = (unsigned long long)std::max(p.num_class, 1) * (unsigned long long)N_global;
        k_bag_draw<<<num_sms * 8, 256, 0, stream>>>(m_total, p.sample_seed, rstate.p, N_global, row_offset, N, K, bag_count.p);
        maxbits.zero(stream);
        k_bag_scale<<<std::max(1, std::min(ceil_div((long long)N * K, 256), num_sms * 8)), 256, 0, stream>>>(gh.p, bag_count.p, (size_t)N * K, maxbits.p);
        launches += 2;
    }
    if (f32) {  // float gradients as they are; root sums in fp64, block partials combined in a fixed order
        k_sum_gh<<<dim3(SUM_BLOCKS, K), 256, 0, stream>>>(gh.p, N, sum_partial.p);
        k_sum_gh_final<<<K, 32, 0, stream>>>(sum_partial.p, SUM_BLOCKS, reinterpret_cast<double *>(root_sum.p));
        launches += 2;
        if (comm && comm->active()) comm->allreduce(root_sum.p, 2 * (size_t)K, Comm::F64, Comm::SUM, stream);
        return;
    }
    if (comm && comm->active()) comm->allreduce(maxbits.p, 2, Comm::U32, Comm::MAX, stream);
    const int blocks = std::max(1, std::min(ceil_div(N, tb), num_sms * 8));
    k_quantize<<<dim3(blocks, K), tb, 0, stream>>>(have_max ? nullptr : gh.p, N, maxbits.p, p.quant_bits, (uint32_t)round, (uint32_t)row_offset,
                                                   ghq.p, root_sum.p, qinfo.p, y.p, ypred.p, logistic, round >= 0 ? rstate.p : nullptr);
    ++launches;
    if (comm && comm->active()) comm->allreduce(root_sum.p, 2 * (size_t)K, Comm::I64, Comm::SUM, stream);
}

// Base score (include/thundergbm/objective/regression_obj.h:35-53 and :95-114): gradients at y_pred = 0,
// w = -sum g / max(sum h, 1e-6) evaluated in double; binary:logistic maps it through sigmoid and logit
// with the host's libm, as the reference does.
void BoosterImpl::init_base_score() {
    base_score = 0;
    if (exact) return;   // include/thundergbm/booster.h:66-73: the reference computes a base score for tree_method = hist only
    if (!(objective == REG_LINEAR || objective == REG_LOGISTIC || objective == BINARY_LOGISTIC)) return;
    gradient(-1);
    unsigned long long hs[2];
    QuantInfo q;
    TGBM_CUDA(cudaMemcpyAsync(hs, root_sum.p, sizeof(hs), cudaMemcpyDeviceToHost, stream));
    TGBM_CUDA(cudaMemcpyAsync(&q, qinfo.p, sizeof(q), cudaMemcpyDeviceToHost, stream));
    TGBM_CUDA(cudaStreamSynchronize(stream));
    float fg, fh;
    if (f32) {
        double d[2];
        memcpy(d, hs, sizeof(d));
        fg = (float)d[0]; fh = (float)d[1];
    } else {
        fg = (float)((double)(long long)hs[0] * q.inv_sg); fh = (float)((double)(long long)hs[1] * q.inv_sh);
    }
    float w = (float)(-(double)fg / std::fmax((double)fh, 1e-6));
    if (objective == BINARY_LOGISTIC) {
        w = 1 / (1 + expf(-w));
        w = -logf(1.0f / w - 1.0f);
    }
    base_score = w;
    p.base_score = w;
    if (N) k_fill<<<std::min(ceil_div(N, 256), num_sms * 8), 256, 0, stream>>>(ypred.p, (size_t)N, w);
}

void BoosterImpl::build_tree(int round, int k) {
    const int tree_index = round * K + k;
    // fp32 mode: the records carry the float gradient pairs themselves (same 8 bytes)
    const int2 *gq = f32 ? reinterpret_cast<const int2 *>(gh.p + (size_t)k * N) : ghq.p + (size_t)k * N;
    const int hist_ctas = std::min(num_sms, HIST_MAX_CTAS);
    k_tree_init<<<ceil_div(n_nodes, 256), 256, 0, stream>>>(nodes.p, n_nodes, root_sum.p + 2 * k, qinfo.p, p.lambda, N,
                                                            seg_begin[0].p, seg_cnt[0].p, gcnt.p, ctl.p, f32 ? 1 : 0);
    k_plan_root<<<1, 1024, 0, stream>>>(seg_begin[0].p, seg_cnt[0].p, gcnt.p, nodes.p, built_right.p, hist_work.p, hist_tile_base.p,
                                        node_tile0[0].p, ctl.p, hist_ctas, hist_cta_off.p, hist_seq.p, depth, tile_node[0].p, part_base.p,
                                        seg_begin[1].p, seg_cnt[1].p, part_group.p, (int)part_group.n);
    launches += 2;
    const int by_hessian = (comm && comm->active()) ? 1 : 0;
    const int colb = p.column_shards > 0 ? 1 : 0;  // candidates, tie rule and child sums of the column-sharded builder
    const int part_ctas = std::max(1, std::min(max_tiles, num_sms * (2048 / PART_THREADS)));
    for (int level = 0; level < depth; ++level) {
        const int cur = level & 1, nxt = cur ^ 1;
        const int nl = 1 << level, pairs = std::max(1, nl / 2);
        const int *idx_in = level == 0 ? nullptr : rec_idx[cur].p;
        const int2 *gh_in = level == 0 ? gq : rec_gh[cur].p;
        // -- histogram of the root / of the smaller child of every pair
        long long *built = level == 0 ? hist_full.p : hist_built.p;
        const int bs = f32 ? f32_stride(pairs) : 1;  // fp32 mode: distance of two cells of the built histograms
        float2 *built_f = bs != 1 ? hist_spread.p : reinterpret_cast<float2 *>(built);
        if (f32) TGBM_CUDA(cudaMemsetAsync(built_f, 0, sizeof(float2) * (size_t)B * pairs * bs, stream));
        else TGBM_CUDA(cudaMemsetAsync(built, 0, sizeof(long long) * 2 * (size_t)B * pairs, stream));
        TimedEvent ev{};
        if (profile_on) {
            cudaEventCreate(&ev.a); cudaEventCreate(&ev.b);
            ev.kind = level == 0 ? 0 : 1;
            cudaEventRecord(ev.a, stream);
        }
        if (f32) {
            const float2 *ghf = reinterpret_cast<const float2 *>(gh_in);
            const int f32_ctas = num_sms * (2048 / F32_THREADS);
            if (sparse) {
                if (level == 0)
                    k_hist_sparse_f32<false><<<f32_ctas, F32_THREADS, 0, stream>>>(sp_row_ptr.p, sp_bin.p, nullptr, ghf, hist_work.p, hist_tile_base.p,
                                                                                   ctl.p, built_f, B, bs);
                else
                    k_hist_sparse_f32<true><<<f32_ctas, F32_THREADS, 0, stream>>>(sp_row_ptr.p, sp_bin.p, idx_in, ghf, hist_work.p, hist_tile_base.p,
                                                                                  ctl.p, built_f, B, bs);
            } else if (level == 0)
                k_hist_f32<false><<<dim3(f32_ctas, G), F32_THREADS, 0, stream>>>(bins.p, Fpad, F, nullptr, ghf, hist_seq.p, ctl.p, cut_ptr.p, built_f, B, bs,
                                                                                 f32_cuts, F <= 256, 0);
            else
                k_hist_f32<true><<<dim3(f32_ctas, G), F32_THREADS, 0, stream>>>(bins.p, Fpad, F, idx_in, ghf, hist_seq.p, ctl.p, cut_ptr.p, built_f, B, bs,
                                                                                f32_cuts, F <= 256, f32_staged ? 1 : 0);
        } else if (sparse) {
            const int sp_ctas = num_sms;
            const size_t sp_smem = (size_t)std::min(B, SPARSE_SMEM_BINS) * 16;
            if (level == 0)
                k_hist_sparse<false><<<sp_ctas, SPARSE_THREADS, sp_smem, stream>>>(sp_row_ptr.p, sp_bin.p, nullptr, gh_in, hist_work.p,
                                                                                   hist_tile_base.p, ctl.p, built, B);
            else
                k_hist_sparse<true><<<sp_ctas, SPARSE_THREADS, sp_smem, stream>>>(sp_row_ptr.p, sp_bin.p, idx_in, gh_in, hist_work.p,
                                                                                  hist_tile_base.p, ctl.p, built, B);
        } else if (level == 0)
            k_hist<false><<<dim3(hist_ctas, G), HIST_THREADS, hist_smem, stream>>>(bins.p, Fpad, F, nullptr, gh_in, hist_cta_off.p, hist_seq.p,
                                                                                   cut_ptr.p, cut_fid.p, built, B, window_rows);
        else
            k_hist<true><<<dim3(hist_ctas, G), HIST_THREADS, hist_smem, stream>>>(bins.p, Fpad, F, idx_in, gh_in, hist_cta_off.p, hist_seq.p,
                                                                                  cut_ptr.p, cut_fid.p, built, B, window_rows);
        if (profile_on) { cudaEventRecord(ev.b, stream); events.push_back(ev); }
        int bs_eval = bs;   // distance of the cells the split search reads
        if (comm && comm->active()) {
            if (f32) {
                // the ranks' sums meet in a compact buffer: spread cells are gathered first (a pass over B x pairs cells)
                float2 *compact = reinterpret_cast<float2 *>(built);
                if (bs != 1) {
                    const size_t cells = (size_t)B * pairs;
                    k_compact_cells<<<std::min(ceil_div(cells, 256), num_sms * 8), 256, 0, stream>>>(built_f, compact, cells, bs);
                    built_f = compact; bs_eval = 1; ++launches;
                }
                comm->allreduce(built_f, 2 * (size_t)B * pairs, Comm::F32, Comm::SUM, stream);
            } else comm->allreduce(built, 2 * (size_t)B * pairs, Comm::I64, Comm::SUM, stream);
        }
        // -- split selection and tree update
        if (f32) {
            const float *parent_f = level == 0 ? nullptr : reinterpret_cast<const float *>(hist_full.p) + full_offset(level - 1);
            float *full_f = reinterpret_cast<float *>(hist_full.p) + full_offset(level);
            const float *bf = reinterpret_cast<const float *>(built_f);
            if (sparse) {
                k_eval_chunk<float><<<dim3(n_chunks, pairs), 64, 0, stream>>>(level, n_chunks, B, chunk_bin0.p, cut_ptr.p, cut_fid.p, nodes.p, built_right.p,
                                                                              bf, parent_f, full_f, qinfo.p, p.min_child_weight, p.lambda, recs.p, bs_eval, ignored_all.p, rstate.p, F, colb);
                k_best_apply<<<nl, 32, 0, stream>>>(level, n_chunks, cut_ptr.p, cut_val.p, recs.p, nodes.p, p.rt_eps, p.lambda, cut_fid.p, 1, colb);
            } else {
                k_eval<float><<<dim3(F, pairs), 64, 0, stream>>>(level, F, B, cut_ptr.p, nodes.p, built_right.p, bf, parent_f, full_f, qinfo.p,
                                                                 p.min_child_weight, p.lambda, recs.p, cut_val.p, p.rt_eps, cut_fid.p, eval_ticket.p, bs_eval,
                                                                 ignored_all.p, rstate.p, colb);
            }
        } else {
        const long long *parent_hist = level == 0 ? nullptr : hist_full.p + full_offset(level - 1);
        if (sparse) {
            k_eval_chunk<long long><<<dim3(n_chunks, pairs), 64, 0, stream>>>(level, n_chunks, B, chunk_bin0.p, cut_ptr.p, cut_fid.p, nodes.p, built_right.p,
                                                                   built, parent_hist, hist_full.p + full_offset(level), qinfo.p,
                                                                   p.min_child_weight, p.lambda, recs.p, 1, ignored_all.p, rstate.p, F, colb);
            k_best_apply<<<nl, 32, 0, stream>>>(level, n_chunks, cut_ptr.p, cut_val.p, recs.p, nodes.p, p.rt_eps, p.lambda, cut_fid.p, 1, colb);
        } else {
            k_eval<long long><<<dim3(F, pairs), 64, 0, stream>>>(level, F, B, cut_ptr.p, nodes.p, built_right.p, built, parent_hist,
                                                      hist_full.p + full_offset(level), qinfo.p, p.min_child_weight, p.lambda, recs.p,
                                                      cut_val.p, p.rt_eps, cut_fid.p, eval_ticket.p, 1, ignored_all.p, rstate.p, colb);
        }
        }
        // -- move the rows (not after the last level: the finished tree is applied by walking it, see k_predict_walk)
        launches += sparse ? 3 : 2;
        if (level == depth - 1) break;
        TimedEvent pv{};
        if (profile_on) { cudaEventCreate(&pv.a); cudaEventCreate(&pv.b); pv.kind = 2; cudaEventRecord(pv.a, stream); }
        if (part_one) {
            // one pass: count, look-back prefix inside every node and scatter; then the plan of the next level
            const int n1 = std::max(N, 1);
            if (sparse)
                k_part_one<true><<<part_ctas, PART_THREADS, 0, stream>>>(level, nodes.p, seg_begin[cur].p, seg_cnt[cur].p, node_tile0[cur].p, tile_node[cur].p,
                                                                         part_base.p, ctl.p, idx_in, gh_in, nullptr, Npad, sp_row_ptr.p, sp_bin.p, cut_ptr.p,
                                                                         part_status.p, part_group.p, seg_begin[nxt].p, seg_cnt[nxt].p, rec_idx[nxt].p, rec_gh[nxt].p, n1, colb);
            else
                k_part_one<false><<<part_ctas, PART_THREADS, 0, stream>>>(level, nodes.p, seg_begin[cur].p, seg_cnt[cur].p, node_tile0[cur].p, tile_node[cur].p,
                                                                          part_base.p, ctl.p, idx_in, gh_in, binsT.p, Npad, nullptr, nullptr, cut_ptr.p,
                                                                          part_status.p, part_group.p, seg_begin[nxt].p, seg_cnt[nxt].p, rec_idx[nxt].p, rec_gh[nxt].p, n1, colb);
            k_plan_next<<<1, 1024, 0, stream>>>(level, seg_begin[nxt].p, seg_cnt[nxt].p, seg_cnt[nxt].p, nodes.p, ctl.p, by_hessian, built_right.p,
                                                hist_work.p, hist_tile_base.p, node_tile0[nxt].p, hist_ctas, hist_cta_off.p, hist_seq.p, depth, tile_node[nxt].p,
                                                part_base.p, seg_begin[cur].p, seg_cnt[cur].p, part_group.p, (int)part_group.n);
            if (profile_on) { cudaEventRecord(pv.b, stream); events.push_back(pv); }
            launches += 2;
            continue;
        }
        if (sparse)
            k_part_count<true><<<part_ctas, PART_THREADS, 0, stream>>>(level, nodes.p, seg_begin[cur].p, seg_cnt[cur].p, node_tile0[cur].p, ctl.p,
                                                                       idx_in, nullptr, Npad, sp_row_ptr.p, sp_bin.p, cut_ptr.p, bits.p, tile_left.p, tile_node[cur].p, colb);
        else
            k_part_count<false><<<part_ctas, PART_THREADS, 0, stream>>>(level, nodes.p, seg_begin[cur].p, seg_cnt[cur].p, node_tile0[cur].p, ctl.p,
                                                                        idx_in, binsT.p, Npad, nullptr, nullptr, cut_ptr.p, bits.p, tile_left.p, tile_node[cur].p, colb);
        k_part_scan<<<1, 1024, 0, stream>>>(level, nodes.p, seg_cnt[cur].p, node_tile0[cur].p, tile_left.p,
                                            seg_begin[nxt].p, seg_cnt[nxt].p, gcnt.p, ctl.p);
        // the next level's plan runs beside the scatter: launched first so that it gets its SM slot, while the
        // scatter leaves 1024 threads' worth of its block slots free
        TGBM_CUDA(cudaEventRecord(ev_scan, stream));
        TGBM_CUDA(cudaStreamWaitEvent(stream2, ev_scan, 0));
        k_plan_next<<<1, 1024, 0, stream2>>>(level, seg_begin[nxt].p, seg_cnt[nxt].p, gcnt.p, nodes.p, ctl.p, by_hessian, built_right.p,
                                             hist_work.p, hist_tile_base.p, node_tile0[nxt].p, hist_ctas, hist_cta_off.p, hist_seq.p, depth, tile_node[nxt].p,
                                             part_base.p, nullptr, nullptr, nullptr, 0);
        TGBM_CUDA(cudaEventRecord(ev_plan, stream2));
        k_part_scatter<<<std::max(1, part_ctas - 1024 / PART_THREADS), PART_THREADS, 0, stream>>>(level, nodes.p, seg_begin[cur].p, seg_cnt[cur].p,
                                                                                node_tile0[cur].p, ctl.p, idx_in, gh_in, bits.p, tile_left.p,
                                                                                seg_begin[nxt].p, rec_idx[nxt].p, rec_gh[nxt].p, tile_node[cur].p);
        TGBM_CUDA(cudaStreamWaitEvent(stream, ev_plan, 0));
        if (profile_on) { cudaEventRecord(pv.b, stream); events.push_back(pv); }
        launches += 4;
    }
    k_prune<<<1, 1024, prune_in_smem ? sizeof(TreeNode) * (size_t)n_nodes : 0, stream>>>(nodes.p, n_nodes, depth, p.gamma, prune_in_smem ? 1 : 0);
    if (N) {
        const size_t per_node = sizeof(WalkNode) + (sparse ? sizeof(WalkSpan) : 0);
        const int in_smem = per_node * (size_t)n_nodes <= 160 * 1024;
        const size_t walk_smem = in_smem ? per_node * (size_t)n_nodes : 0;
        float *yp = ypred.p + (size_t)k * N;
        int *nid_out = p.keep_nid ? nid_keep.p + (size_t)tree_index * N : nullptr;
        // One tree per round and a pointwise objective: the walk also adds up the round's metric and finds the maxima
        // of the next round's gradients (grid and order of additions are those of k_metric_partial).
        const bool fuse = K == 1 && (objective == REG_LINEAR || objective == REG_LOGISTIC || objective == BINARY_LOGISTIC);
        const int walk_ctas = fuse ? metric_blocks() : std::min(ceil_div(N, 256), num_sms * 8);
        const int fo = fuse ? objective : -1;
        if (fuse) maxbits.zero(stream);
        if (sparse)
            k_predict_walk<2><<<walk_ctas, 256, walk_smem, stream>>>(nodes.p, n_nodes, in_smem, nullptr, Fpad, sp_row_ptr.p, sp_bin.p, cut_ptr.p, N,
                                                                     p.learning_rate, yp, nid_out, y.p, fo, metric_partial.p, maxbits.p, colb);
        else if (Fpad == 32)
            k_predict_walk<0><<<walk_ctas, 256, walk_smem, stream>>>(nodes.p, n_nodes, in_smem, bins.p, Fpad, nullptr, nullptr, cut_ptr.p, N,
                                                                     p.learning_rate, yp, nid_out, y.p, fo, metric_partial.p, maxbits.p, colb);
        else
            k_predict_walk<1><<<walk_ctas, 256, walk_smem, stream>>>(nodes.p, n_nodes, in_smem, bins.p, Fpad, nullptr, nullptr, cut_ptr.p, N,
                                                                     p.learning_rate, yp, nid_out, y.p, fo, metric_partial.p, maxbits.p, colb);
        grad_max_ready = metric_partial_ready = fuse;
    }
    launches += 2;
    k_store_tree<<<std::min(ceil_div(n_nodes, 256), 64), 256, 0, stream>>>(nodes.p, model.p, n_nodes, K, k, rstate.p);
    ++launches;
}

void BoosterImpl::round_metric(int round) {
    const int log_len = (int)qinfo_log.n;
    if (need_group_file(objective)) {
        rank.metric(objective, ypred.p, nullptr, comm, N_global, stream);
        k_round_end<<<1, 32, 0, stream>>>(objective, rank.sum.p, rank.n_group_total, metric.p, qinfo.p, qinfo_log.p, log_len, rstate.p);
        ++launches;
        return;
    }
    const int blocks = metric_blocks();
    if (!metric_partial_ready) {  // else the walk that applied the round's tree has left the partial sums
        k_metric_partial<<<blocks, 256, 0, stream>>>(objective, y.p, ypred.p, N, K, metric_partial.p);
        ++launches;
    }
    metric_partial_ready = false;
    k_metric_sum<<<1, 32, 0, stream>>>(metric_partial.p, blocks, metric_sum.p);
    if (comm && comm->active()) comm->allreduce(metric_sum.p, 1, Comm::F64, Comm::SUM, stream);
    k_round_end<<<1, 32, 0, stream>>>(objective, metric_sum.p, N_global, metric.p, qinfo.p, qinfo_log.p, log_len, rstate.p);
    launches += 2;
}

// One boosting round.  From the second round on the launch sequence no longer changes (which kernels run is decided
// by the objective and by flags that have reached their steady state; everything that depends on the data is decided
// on the device), so it is captured once into a CUDA graph and replayed: one launch per round instead of ~60, no
// gaps between the small per-level kernels.  Not with profiling events or a kept row->node table.  With a communicator
// the NCCL calls of the round are captured with it (every rank captures and replays the same sequence).
void BoosterImpl::run_round(int round) {
    auto direct = [&]() {
        gradient(round);
        for (int k = 0; k < K; ++k) {
            if (exact) build_tree_exact(round, k);
            else build_tree(round, k);
        }
        round_metric(round);
    };
    static const bool graph_with_comm = getenv("TGBM_NO_GRAPH_COMM") == nullptr;  // the round's collectives are captured with it
    // Ranks that are threads of ONE process do not replay graphs: instantiating a graph allocates device memory, and with
    // peer access enabled such a call can wait for the other devices of the process -- whose collective kernels may
    // already be waiting for this rank's.  (Between processes there is no such coupling.)
    const bool in_process_group = comm && comm->active() && comm->host;
    const bool graph_ok = graphs_allowed && round >= 1 && !profile_on && !p.keep_nid && !in_process_group &&
                          (graph_with_comm || !(comm && comm->active()));
    if (!graph_ok) { direct(); return; }
    if (!round_exec) {
        const long long before = launches;
        TGBM_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        bool ok = true;
        try { direct(); } catch (...) { ok = false; }
        cudaGraph_t g = nullptr;
        const cudaError_t rc = cudaStreamEndCapture(stream, &g);
        round_graph_launches = launches - before;
        launches = before;
        if (!ok || rc != cudaSuccess || !g) {  // fall back to plain launches for good
            if (g) cudaGraphDestroy(g);
            cudaGetLastError();
            graphs_allowed = false;
            TGBM_CHECK(ok, "capturing a boosting round failed");
            direct();
            return;
        }
        round_graph = g;
        TGBM_CUDA(cudaGraphInstantiate(&round_exec, round_graph, 0));
    }
    TGBM_CUDA(cudaGraphLaunch(round_exec, stream));
    launches += round_graph_launches;
}

void Booster::boost(int n_rounds) {
    BoosterImpl &m = *impl_;
    TGBM_CHECK(m.rounds + n_rounds <= m.p.n_trees, "boost() beyond n_trees");
    for (int i = 0; i < n_rounds; ++i) {
        m.run_round(m.rounds);
        ++m.rounds;
    }
    TGBM_CUDA(cudaGetLastError());
}

void Booster::sync() {
    if (impl_->comm && impl_->comm->active()) impl_->comm->wait(impl_->stream);  // bounded: a rank may have left
    else TGBM_CUDA(cudaStreamSynchronize(impl_->stream));
    TGBM_CUDA(cudaGetLastError());
    // bounded waits inside the kernels (look-back of the single-pass partition, bulk-copy barriers of the fp32 histogram
    // kernel) report here instead of spinning: the results of the run are not to be trusted
    if (impl_->ctl.p) {
        int err = 0;
        TGBM_CUDA(cudaMemcpy(&err, reinterpret_cast<const char *>(impl_->ctl.p) + offsetof(TreeCtl, error), sizeof(int), cudaMemcpyDeviceToHost));
        TGBM_CHECK(err == 0, "a bounded wait inside a kernel ran out (code " + std::to_string(err) + "); the trees of this run are invalid");
    }
}

int Booster::rounds_done() const { return impl_->rounds; }
int Booster::trees_per_round() const { return impl_->K; }
int Booster::n_nodes() const { return impl_->n_nodes; }
int Booster::num_class() const { return impl_->num_class; }
float Booster::base_score() const { return impl_->base_score; }
int Booster::n_bins() const { return impl_->B; }
int Booster::n_features() const { return impl_->F; }
std::string Booster::tree_method() const { return impl_->p.tree_method; }
int Booster::fpad() const { return impl_->Fpad; }
cudaStream_t Booster::stream() const { return impl_->stream; }
void Booster::set_profile(bool on) {
    BoosterImpl &m = *impl_;
    if (on && !m.profile_on && m.ctl.p) {  // the byte counters of the plan kernels run all the time: remember where profiling starts
        sync();
        TGBM_CUDA(cudaMemcpy(&m.stat_base, m.ctl.p, sizeof(TreeCtl), cudaMemcpyDeviceToHost));
    }
    m.profile_on = on;
}

HistProfile Booster::profile() {
    BoosterImpl &m = *impl_;
    sync();
    HistProfile r;
    for (auto &e : m.events) {
        float ms = 0;
        cudaEventElapsedTime(&ms, e.a, e.b);
        if (e.kind == 2) { r.partition_ms += ms; r.partition_launches += 4; }
        else {
            r.hist_ms += ms; r.hist_launches += 1;
            if (e.kind == 0) { r.hist_root_ms += ms; r.hist_root_launches += 1; }
        }
    }
    // the timed events have been read: their times move into running totals and the events are destroyed, so that a
    // long profiled run does not pile them up
    for (auto &e : m.events) { cudaEventDestroy(e.a); cudaEventDestroy(e.b); }
    m.events.clear();
    m.profile_acc.hist_ms += r.hist_ms; m.profile_acc.hist_launches += r.hist_launches;
    m.profile_acc.hist_root_ms += r.hist_root_ms; m.profile_acc.hist_root_launches += r.hist_root_launches;
    m.profile_acc.partition_ms += r.partition_ms; m.profile_acc.partition_launches += r.partition_launches;
    r = m.profile_acc;
    TreeCtl c;
    TGBM_CUDA(cudaMemcpy(&c, m.ctl.p, sizeof(c), cudaMemcpyDeviceToHost));
    // algorithmic bytes: rows * (F bin bytes + 8 gradient bytes [+ 4 row index]) + histograms * B * 16 written
    // per row: its bin ids (F bytes dense; 4 bytes per stored value + a row pointer in the CSR layout), 8 gradient bytes
    const double row_bytes = m.sparse ? 4.0 * (double)m.nnz_local / std::max(1, m.N) + 4.0 : (double)m.F;
    const TreeCtl &c0 = m.stat_base;
    r.hist_root_bytes = (double)(c.stat_rows_root - c0.stat_rows_root) * (row_bytes + 8);
    r.hist_bytes = r.hist_root_bytes + (double)(c.stat_rows_gather - c0.stat_rows_gather) * (row_bytes + 8 + 4) +
                   (double)(c.stat_hists - c0.stat_hists) * m.B * (m.f32 ? 8.0 : 16.0);
    r.partition_bytes = (double)(c.stat_part_rows - c0.stat_part_rows) * (4 + 1 + 4);
    r.hist_rows = (long long)((c.stat_rows_root - c0.stat_rows_root) + (c.stat_rows_gather - c0.stat_rows_gather));
    r.kernel_launches = m.launches;
    return r;
}

std::vector<std::vector<Tree>> Booster::get_model() {
    BoosterImpl &m = *impl_;
    sync();
    std::vector<TreeNode> h((size_t)m.rounds * m.K * m.n_nodes);
    if (!h.empty()) TGBM_CUDA(cudaMemcpy(h.data(), m.model.p, sizeof(TreeNode) * h.size(), cudaMemcpyDeviceToHost));
    std::vector<std::vector<Tree>> out(m.rounds);
    for (int r = 0; r < m.rounds; ++r) {
        out[r].resize(m.K);
        for (int k = 0; k < m.K; ++k) {
            const TreeNode *src = h.data() + ((size_t)r * m.K + k) * m.n_nodes;
            out[r][k].nodes.assign(src, src + m.n_nodes);
        }
    }
    return out;
}

template <typename T>
static std::vector<T> to_host(const T *p, size_t n) {
    std::vector<T> h(n);
    if (n) TGBM_CUDA(cudaMemcpy(h.data(), p, sizeof(T) * n, cudaMemcpyDeviceToHost));
    return h;
}

std::vector<float> Booster::get_metrics() { sync(); return to_host(impl_->metric.p, impl_->rounds); }
std::vector<float> Booster::get_ypred() { sync(); return to_host(impl_->ypred.p, (size_t)impl_->N * impl_->K); }
std::vector<float> Booster::get_cut_val() const { return impl_->h_cut_val; }
std::vector<int> Booster::get_cut_ptr() const { return impl_->h_cut_ptr; }
std::vector<unsigned char> Booster::get_bins() {
    sync();
    TGBM_CHECK(!impl_->sparse, "the booster holds the CSR layout: use get_bins_csr");
    return to_host(impl_->bins.p, (size_t)impl_->N * impl_->Fpad);
}
std::vector<int> Booster::get_bins_csr() {
    sync();
    TGBM_CHECK(impl_->sparse, "the booster holds the dense layout: use get_bins");
    return to_host(impl_->sp_bin.p, (size_t)impl_->nnz_local);
}
bool Booster::is_sparse() const { return impl_->sparse; }
std::vector<int> Booster::get_nid() {
    sync();
    if (!impl_->p.keep_nid) return {};
    return to_host(impl_->nid_keep.p, (size_t)impl_->N * impl_->K * impl_->rounds);
}
std::vector<long long> Booster::get_root_hist() {
    sync();
    TGBM_CHECK(!impl_->f32, "fp32 mode keeps float histograms: use get_root_hist_f32");
    return to_host(impl_->hist_full.p, (size_t)impl_->B * 2);
}
std::vector<float> Booster::get_root_hist_f32() {
    sync();
    TGBM_CHECK(impl_->f32, "exact mode keeps integer histograms: use get_root_hist");
    return to_host(reinterpret_cast<const float *>(impl_->hist_full.p), (size_t)impl_->B * 2);
}
std::vector<double> Booster::get_quant_scale() {
    sync();
    auto q = to_host(impl_->qinfo_log.p, impl_->rounds);
    std::vector<double> r;
    for (auto &v : q) { r.push_back(v.sg); r.push_back(v.sh); }
    return r;
}

}  // namespace tgbm
