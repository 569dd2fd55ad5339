// extern "C" boundary of libthundergbm.so; declarations and reference citations in include/thundergbm.h
#include <algorithm>
#include <chrono>
#include <climits>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>

#include "../../include/thundergbm.h"
#include "tgbm_booster.h"
#include "tgbm_device.cuh"

// the opaque C handle is the C++ tree container
struct Tree : tgbm::Tree {};
struct TgbmComm { tgbm::Comm *c; };
struct TgbmBooster {
    tgbm::Booster *b = nullptr;
    tgbm::GBMParam param;
    std::vector<float> label;
    int n_rows = 0;
    ~TgbmBooster() { delete b; }  // also when init() throws half way through tgbm_booster_create
};

namespace {
thread_local std::string g_err;

template <typename F>
int guard(F &&f) {
    int rc = 0;
    try {
        g_err.clear();
        f();
    } catch (const std::exception &e) {
        g_err = e.what();
        if (tgbm::verbosity() >= 1) fprintf(stderr, "thundergbm: %s\n", g_err.c_str());
        rc = 1;
    }
    tgbm::dev_trim();   // what the call released stays mapped for the next one, up to the pools' limit
    return rc;
}

std::vector<std::vector<tgbm::Tree>> wrap_model(::Tree *model, int n_trees, int per_iter) {
    TGBM_CHECK(model != nullptr, "model is null!");
    std::vector<std::vector<tgbm::Tree>> m(n_trees);
    for (int i = 0; i < n_trees; ++i)
        for (int j = 0; j < per_iter; ++j) m[i].push_back(model[(size_t)i * per_iter + j]);
    return m;
}

::Tree *unwrap_model(const std::vector<std::vector<tgbm::Tree>> &m) {
    const size_t per = m.empty() ? 0 : m[0].size();
    ::Tree *out = new ::Tree[std::max<size_t>(1, m.size() * per)];
    for (size_t i = 0; i < m.size(); ++i)
        for (size_t j = 0; j < per; ++j) out[i * per + j].nodes = m[i][j].nodes;
    return out;
}

// TreeTrainer::train (src/thundergbm/trainer.cu:18-57) for the histogram path
std::vector<std::vector<tgbm::Tree>> train(tgbm::GBMParam &p, const tgbm::DataSet &ds, const tgbm::Comm *comm) {
    TGBM_CHECK(p.tree_method == "hist" || p.tree_method == "auto" || p.tree_method == "exact", "unknown tree_method " + p.tree_method);
    const bool timing = getenv("TGBM_TIMING") != nullptr;  // phase times on stderr
    auto t_mark = std::chrono::steady_clock::now();
    auto lap = [&](const char *what) {
        if (!timing) return;
        const auto t = std::chrono::steady_clock::now();
        fprintf(stderr, "[tgbm train] %-26s %8.1f ms\n", what, std::chrono::duration<double, std::milli>(t - t_mark).count());
        t_mark = t;
    };
    std::vector<std::vector<tgbm::Tree>> result;
    {
    tgbm::Booster booster(p, comm);
    booster.init(ds);  // counts the features when the data set has not, and resolves tree_method=auto (trainer.cu:19-23)
    p.tree_method = booster.tree_method();
    lap("init");
    const auto t0 = std::chrono::high_resolution_clock::now();
    booster.boost(p.n_trees);
    booster.sync();
    const auto t1 = std::chrono::high_resolution_clock::now();
    lap("boost");
    const auto metrics = booster.get_metrics();
    if (!comm || comm->rank == 0) {
        for (size_t i = 0; i < metrics.size(); ++i)  // include/thundergbm/booster.h:91-92
            tgbm::log_info("[%zu/%d] %s = %g", i + 1, p.n_trees, tgbm::metric_name(tgbm::objective_from_name(p.objective)), metrics[i]);
        tgbm::log_info("training time = %g", std::chrono::duration<float>(t1 - t0).count());  // trainer.cu:50
    }
    p.base_score = booster.base_score();
    p.num_class = booster.num_class();
    p.tree_per_rounds = booster.trees_per_round();
    result = booster.get_model();
    lap("metrics + model read-back");
    }
    lap("booster teardown");
    return result;
}

// n_device > 1 through the reference's own entry points (include/thundergbm/booster.h:39-64 runs one OpenMP thread per
// GPU inside the process).  Here too: one host thread per GPU, devices 0 .. n_device-1, each with a contiguous block
// of the rows (query groups stay whole), an NCCL communicator between them and a host-side meeting point
// (tgbm::HostGroup) so that a rank that fails takes the others with it instead of leaving them in a collective.
// The rows are sharded, not the columns, and every rank builds the same trees; rank 0's copy is returned.
// The communicators of an in-process group outlive the call: setting one up costs a few hundred milliseconds, a
// 100-round training on eight GPUs little more.  One set per device count, used by one call at a time, dropped when a
// call fails (its communicators may have been aborted), never torn down at process exit.  TGBM_NO_COMM_CACHE=1 makes
// every call build and destroy its own.
std::mutex g_group_mutex;
std::map<int, std::vector<tgbm::Comm *>> g_group_comms;

std::vector<std::vector<tgbm::Tree>> train_in_process(tgbm::GBMParam &p, const tgbm::DataSet &ds, int n_dev) {
    std::lock_guard<std::mutex> one_call_at_a_time(g_group_mutex);
    const bool keep_comms = getenv("TGBM_NO_COMM_CACHE") == nullptr;
    std::vector<tgbm::Comm *> comms(n_dev, nullptr);
    {
        auto it = g_group_comms.find(n_dev);
        if (it != g_group_comms.end()) { comms = it->second; g_group_comms.erase(it); }
    }
    int avail = 0;
    TGBM_CUDA(cudaGetDeviceCount(&avail));
    TGBM_CHECK(n_dev <= avail, "n_device = " + std::to_string(n_dev) + " but only " + std::to_string(avail) + " GPU(s) are visible");
    int caller_dev = 0;
    TGBM_CUDA(cudaGetDevice(&caller_dev));
    unsigned char id[128];
    tgbm::comm_get_unique_id(id);
    double group_timeout_s = 120.0;  // how long a rank waits for the others at a meeting point (TGBM_GROUP_TIMEOUT_S)
    if (const char *e = getenv("TGBM_GROUP_TIMEOUT_S")) group_timeout_s = atof(e) > 0 ? atof(e) : group_timeout_s;
    auto group = std::make_shared<tgbm::HostGroup>(n_dev, group_timeout_s);
    // row blocks: rows n*r/W, moved to the next query-group boundary when there are groups
    std::vector<int> row_lo(n_dev + 1, 0), grp_lo(n_dev + 1, 0);
    {
        std::vector<long long> gend;
        long long acc = 0;
        for (int g : ds.group) { acc += g; gend.push_back(acc); }
        for (int r = 1; r < n_dev; ++r) {
            long long want = (long long)ds.n_rows * r / n_dev;
            if (!gend.empty()) {
                const size_t gi = std::lower_bound(gend.begin(), gend.end(), want) - gend.begin();
                grp_lo[r] = (int)std::min(gi + 1, gend.size());
                want = grp_lo[r] ? gend[grp_lo[r] - 1] : 0;
            }
            row_lo[r] = (int)want;
        }
        row_lo[n_dev] = ds.n_rows;
        grp_lo[n_dev] = (int)ds.group.size();
    }
    std::vector<std::string> errors(n_dev);
    std::vector<std::vector<tgbm::Tree>> result;
    tgbm::GBMParam p0 = p;
    std::vector<std::thread> threads;
    for (int r = 0; r < n_dev; ++r)
        threads.emplace_back([&, r] {
            tgbm::Comm *&c = comms[r];
            try {
                TGBM_CUDA(cudaSetDevice(r));
                if (!c) c = tgbm::comm_create(id, r, n_dev);
                c->host = group;
                const int lo = row_lo[r], hi = row_lo[r + 1];
                tgbm::DataSet shard;
                shard.n_rows = hi - lo;
                shard.n_features = ds.n_features;
                shard.row_ptr.resize(hi - lo + 1);
                for (int i = lo; i <= hi; ++i) shard.row_ptr[i - lo] = ds.rp[i] - ds.rp[lo];
                shard.rp = shard.row_ptr.data();
                shard.ci = ds.ci + ds.rp[lo];
                shard.vv = ds.vv + ds.rp[lo];
                const float *labels = ds.yv ? ds.yv : ds.y.data();
                shard.yv = labels ? labels + lo : nullptr;
                shard.labels_raw = ds.labels_raw;
                shard.label = ds.label;
                shard.group.assign(ds.group.begin() + grp_lo[r], ds.group.begin() + grp_lo[r + 1]);
                tgbm::GBMParam pr = p0;
                auto m = train(pr, shard, c);
                if (r == 0) { result = std::move(m); p = pr; }
            } catch (const std::exception &e) {
                errors[r] = e.what();
                group->abandon();
            }
        });
    for (auto &t : threads) t.join();
    bool failed = false;
    for (const auto &e : errors) failed = failed || !e.empty();
    if (failed || !keep_comms) {
        std::vector<std::thread> closers;   // every rank leaves its communicator on a thread of its own, as it joined it
        for (int r = 0; r < n_dev; ++r)
            closers.emplace_back([&, r] {
                if (!comms[r]) return;
                cudaSetDevice(r);
                comms[r]->host.reset();
                tgbm::comm_destroy(comms[r]);
            });
        for (auto &t : closers) t.join();
    } else {
        for (auto *c : comms) c->host.reset();
        g_group_comms[n_dev] = comms;
    }
    cudaSetDevice(caller_dev);
    // a rank's own failure explains more than the "another rank failed" of its peers
    std::string first, own;
    for (int r = 0; r < n_dev; ++r) {
        if (errors[r].empty()) continue;
        if (first.empty()) first = errors[r];
        if (own.empty() && errors[r].find("another rank") == std::string::npos) own = "rank " + std::to_string(r) + ": " + errors[r];
    }
    if (!first.empty()) throw tgbm::Error(own.empty() ? first : own);
    return result;
}

// distinct integer labels over all ranks (DataSet::group_label applied to the union); the rows keep the caller's
// label values, the booster maps them to class indices on the device
void group_label_global(tgbm::DataSet &ds, const float *label, tgbm::GBMParam &p, const tgbm::Comm *comm) {
    constexpr int CAP = 4096;
    // Failures of this rank alone (too many labels, no device memory) travel WITH the all-gather as a marker in slot 0,
    // so that every rank leaves together instead of this one alone before the collective.
    std::string local_err;
    std::vector<int> padded(CAP, INT_MAX);
    tgbm::DevBuf<int> d_in, d_out;
    try {
        ds.distinct_labels(label, (size_t)ds.n_rows);
        TGBM_CHECK((int)ds.label.size() <= CAP, "more than 4096 distinct labels");
        for (size_t i = 0; i < ds.label.size(); ++i) padded[i] = (int)ds.label[i];
        d_in.alloc(CAP); d_out.alloc((size_t)CAP * comm->world);
    } catch (const std::exception &e) { local_err = e.what(); }
    comm->agree(local_err, "grouping its labels", nullptr);
    TGBM_CUDA(cudaMemcpy(d_in.p, padded.data(), sizeof(int) * CAP, cudaMemcpyHostToDevice));
    comm->allgather(d_in.p, d_out.p, CAP, tgbm::Comm::I32, nullptr);
    std::vector<int> all((size_t)CAP * comm->world);
    comm->wait(nullptr);
    TGBM_CUDA(cudaMemcpy(all.data(), d_out.p, sizeof(int) * all.size(), cudaMemcpyDeviceToHost));
    std::sort(all.begin(), all.end());
    all.erase(std::unique(all.begin(), all.end()), all.end());
    if (!all.empty() && all.back() == INT_MAX) all.pop_back();
    ds.label.clear();
    for (int v : all) ds.label.push_back((float)v);
    ds.labels_raw = true;
    p.num_class = (int)ds.label.size();
}

tgbm::GBMParam param_from_c(const TgbmParam *cp) {
    tgbm::GBMParam p;
    p.depth = cp->depth; p.n_trees = cp->n_trees; p.max_num_bin = cp->max_num_bin; p.num_class = cp->num_class;
    p.min_child_weight = cp->min_child_weight; p.lambda = cp->lambda; p.gamma = cp->gamma; p.learning_rate = cp->learning_rate;
    p.objective = cp->objective ? cp->objective : "reg:linear";
    p.quant_bits = cp->quant_bits; p.keep_nid = cp->keep_nid; p.verbose = cp->verbose; p.rank_seed = cp->rank_seed;
    p.hist_mode = cp->hist_mode;
    p.bagging = cp->bagging != 0; p.column_sampling_rate = cp->column_sampling_rate; p.sample_seed = cp->sample_seed;
    p.column_shards = cp->column_shards;
    p.tree_method = cp->exact_builder ? "exact" : "hist";
    return p;
}
}  // namespace

namespace tgbm {
std::vector<std::vector<Tree>> train_model(GBMParam &p, const DataSet &ds) {
    TGBM_CHECK(p.n_device >= 1, "n_device must be at least 1");
    // TGBM_COLUMN_BUILDER=1: n_device = D > 1 also selects what the reference's D-device builder computes
    if (const char *e = getenv("TGBM_COLUMN_BUILDER"))
        if (*e && strcmp(e, "0") && p.n_device > 1 && p.column_shards == 0) p.column_shards = p.n_device;
    if (p.n_device > 1) {
        // the exact builder (asked for, or what "auto" means above 20000 columns, trainer.cu:19-23) runs on one GPU
        bool exact = p.tree_method == "exact";
        if (p.tree_method == "auto") exact = (ds.n_features >= 0 ? ds.n_features : ds.count_features()) > 20000;
        if (exact) {
            log_info("tree_method = exact trains on one GPU; n_device = %d is not used", p.n_device);
            return train(p, ds, nullptr);
        }
    }
    return p.n_device > 1 ? train_in_process(p, ds, p.n_device) : train(p, ds, nullptr);
}
void set_last_error(const std::string &msg) { g_err = msg; }
int default_hist_mode() {
    const char *e = getenv("TGBM_HIST_MODE");
    if (!e || !*e) return 0;
    const int m = hist_mode_from_name(e);
    TGBM_CHECK(m >= 0, std::string("TGBM_HIST_MODE must be fp32 or exact, not ") + e);
    return m;
}
}  // namespace tgbm

extern "C" {

const char *tgbm_last_error(void) { return g_err.c_str(); }

void set_logger(int verbose) { tgbm::set_verbosity(verbose); }

void sparse_train_scikit(int row_size, float *val, int *row_ptr, int *col_ptr, float *label, int depth, int n_trees,
                         int n_device, float min_child_weight, float lambda, float gamma, int max_num_bin, int verbose,
                         float column_sampling_rate, int bagging, int n_parallel_trees, float learning_rate,
                         char *obj_type, int *num_class, char *tree_method, ::Tree **model, int *tree_per_iter,
                         float *group_label, int *group, int num_group) {
    if (model) *model = nullptr;
    guard([&] {
        tgbm::GBMParam p;
        p.depth = depth; p.n_trees = n_trees; p.n_device = n_device; p.min_child_weight = min_child_weight;
        p.lambda = lambda; p.gamma = gamma; p.max_num_bin = max_num_bin; p.verbose = verbose;
        p.column_sampling_rate = column_sampling_rate; p.bagging = bagging != 0; p.n_parallel_trees = n_parallel_trees;
        p.learning_rate = learning_rate; p.objective = obj_type; p.num_class = *num_class; p.tree_method = tree_method;
        p.rt_eps = 1e-6f; p.tree_per_rounds = 1;
        p.hist_mode = tgbm::default_hist_mode();
        set_logger(verbose);
        TGBM_CHECK(n_device >= 1, "n_device must be at least 1");
        tgbm::DataSet ds;
        ds.load_from_sparse(row_size, val, row_ptr, col_ptr, label, group, num_group, p, /*lazy=*/true);
        tgbm::log_info("#instances = %d", ds.n_rows);
        *num_class = p.num_class;
        auto m = tgbm::train_model(p, ds);
        *num_class = p.num_class;
        *tree_per_iter = m.empty() ? 1 : (int)m[0].size();
        TGBM_CHECK((int)m.size() == n_trees, "trained fewer rounds than requested");
        *model = unwrap_model(m);
        for (size_t i = 0; i < ds.label.size(); ++i) group_label[i] = ds.label[i];
    });
}

void sparse_predict_scikit(int row_size, float *val, int *row_ptr, int *col_ptr, float *y_pred, ::Tree **model,
                           int n_trees, int trees_per_iter, char *objective, int num_class, float learning_rate,
                           float *group_label, int *group, int num_group, int verbose) {
    guard([&] {
        tgbm::GBMParam p;
        p.objective = objective; p.learning_rate = learning_rate; p.num_class = num_class;
        tgbm::DataSet ds;
        ds.load_from_sparse(row_size, val, row_ptr, col_ptr, nullptr, group, num_group, p);
        set_logger(verbose);
        ds.label.clear();
        if (group_label) for (int i = 0; i < num_class; ++i) ds.label.push_back(group_label[i]);
        TGBM_CHECK(model && *model, "model is null!");
        auto m = wrap_model(*model, n_trees, trees_per_iter);
        std::vector<float> y;
        tgbm::predict_raw(ds, m, learning_rate, /*base_score: never set on this path, scikit_tgbm.cpp:87-90*/ 0.f, y);
        tgbm::predict_transform(tgbm::objective_from_name(p.objective), num_class, ds.label, row_size, y);
        std::copy(y.begin(), y.end(), y_pred);
    });
}

void save(char *model_path, char *objective, float learning_rate, int num_class, int n_trees, int trees_per_iter,
          ::Tree **model, float *group_label) {
    guard([&] {
        tgbm::GBMParam p;
        p.objective = objective; p.learning_rate = learning_rate; p.num_class = num_class; p.n_trees = n_trees;
        p.base_score = 0;  // scikit_tgbm.cpp:125-129 leaves it at its default
        TGBM_CHECK(model && *model, "model is null!");
        auto m = wrap_model(*model, n_trees, trees_per_iter);
        std::vector<float> label;
        if (num_class != 1 && group_label) label.assign(group_label, group_label + num_class);
        tgbm::save_model(model_path, p, m, label);
    });
}

void load_model(char *model_path, float *learning_rate, int *num_class, int *n_trees, int *trees_per_iter, ::Tree **model) {
    if (model) *model = nullptr;
    guard([&] {
        tgbm::GBMParam p;
        std::vector<std::vector<tgbm::Tree>> m;
        std::vector<float> label;
        tgbm::load_model(model_path, p, m, label);
        *learning_rate = p.learning_rate; *num_class = p.num_class; *n_trees = p.n_trees;
        *trees_per_iter = m.empty() ? 1 : (int)m[0].size();
        TGBM_CHECK((int)m.size() == *n_trees, "model file: n_trees does not match the number of rounds stored");
        *model = unwrap_model(m);
    });
}

void load_config(char *model_path, float *group_label) {
    guard([&] {
        tgbm::GBMParam p;
        std::vector<std::vector<tgbm::Tree>> m;
        std::vector<float> label;
        tgbm::load_model(model_path, p, m, label);
        for (size_t i = 0; i < label.size(); ++i) group_label[i] = label[i];
    });
}

void get_n_nodes(::Tree **model, int *n_nodes, int n_trees, int tree_per_iter) {
    guard([&] {
        TGBM_CHECK(model && *model, "model is null!");
        for (int i = 0; i < n_trees * tree_per_iter; ++i) n_nodes[i] = (int)(*model)[i].nodes.size();
    });
}

void get_a_tree(::Tree **model, int tree_id, int n_nodes, int *children_left, int *children_right, int *children_default,
                int *features, float *thresholds, float *values, float *node_sample_weights) {
    guard([&] {
        TGBM_CHECK(model && *model, "model is null!");
        const auto &t = (*model)[tree_id];
        TGBM_CHECK(n_nodes == (int)t.nodes.size(), "n_nodes does not match the tree");
        for (int i = 0; i < n_nodes; ++i) {
            const tgbm::TreeNode &n = t.nodes[i];
            children_left[i] = n.lch_index;
            children_right[i] = n.rch_index;
            children_default[i] = n.default_right ? n.rch_index : n.lch_index;
            if (n.is_leaf) { children_left[i] = children_right[i] = children_default[i] = -1; values[i] = n.base_weight; }
            else values[i] = 0;
            features[i] = n.split_feature_id;
            thresholds[i] = n.split_value;
            node_sample_weights[i] = n.sum_h;
        }
    });
}

void model_free(::Tree **model) {
    if (model && *model) { delete[] *model; *model = nullptr; }
}

void train_R(int *depth, int *n_trees, int *n_gpus, int *verbose, int *profiling, char **data, int *max_num_bin,
             double *column_sampling_rate, int *bagging, int *n_parallel_trees, double *learning_rate, char **objective,
             int *num_class, int *min_child_weight, double *lambda_tgbm, double *gamma, char **tree_method, char **model_out) {
    guard([&] {
        tgbm::GBMParam p;
        p.depth = *depth; p.n_trees = *n_trees; p.n_device = *n_gpus; p.verbose = *verbose; p.profiling = *profiling != 0;
        p.path = data[0]; p.max_num_bin = *max_num_bin; p.column_sampling_rate = (float)*column_sampling_rate;
        p.bagging = *bagging != 0; p.n_parallel_trees = *n_parallel_trees; p.learning_rate = (float)*learning_rate;
        p.objective = objective[0]; p.num_class = *num_class; p.min_child_weight = (float)*min_child_weight;
        p.lambda = (float)*lambda_tgbm; p.gamma = (float)*gamma; p.tree_method = tree_method[0];
        p.hist_mode = tgbm::default_hist_mode();
        set_logger(*verbose);
        tgbm::DataSet ds;
        ds.load_from_file(p.path, p);
        auto m = tgbm::train_model(p, ds);
        tgbm::save_model(model_out[0], p, m, ds.label);
    });
}

void predict_R(char **data, char **model_in, int *verbose) {
    guard([&] {
        set_logger(*verbose);
        tgbm::GBMParam p;
        std::vector<std::vector<tgbm::Tree>> m;
        std::vector<float> label;
        tgbm::load_model(model_in[0], p, m, label);
        tgbm::DataSet ds;
        ds.load_from_file(data[0], p);
        std::vector<float> y;
        tgbm::predict_raw(ds, m, p.learning_rate, p.base_score, y);
        const int o = tgbm::objective_from_name(p.objective);
        tgbm::log_info("%s = %g", tgbm::metric_name(o), tgbm::metric_score(o, ds, p.num_class, y));
    });
}

// ------------------------------------------------------------------------------------ part 2
void tgbm_default_param(TgbmParam *p) {
    tgbm::GBMParam d;
    p->depth = d.depth; p->n_trees = d.n_trees; p->max_num_bin = d.max_num_bin; p->num_class = d.num_class;
    p->min_child_weight = d.min_child_weight; p->lambda = d.lambda; p->gamma = d.gamma; p->learning_rate = d.learning_rate;
    p->objective = "reg:linear"; p->quant_bits = d.quant_bits; p->keep_nid = 0; p->verbose = 0; p->profile = 0; p->rank_seed = 0;
    p->hist_mode = tgbm::default_hist_mode();
    p->bagging = 0; p->column_sampling_rate = 1.f; p->sample_seed = 0; p->column_shards = 0; p->exact_builder = 0;
}

int tgbm_comm_unique_id(unsigned char id[128]) { return guard([&] { tgbm::comm_get_unique_id(id); }); }
TgbmComm *tgbm_comm_create(const unsigned char id[128], int rank, int world) {
    TgbmComm *c = nullptr;
    guard([&] { c = new TgbmComm{tgbm::comm_create(id, rank, world)}; });
    return c;
}
void tgbm_comm_destroy(TgbmComm *c) {
    if (!c) return;
    tgbm::comm_destroy(c->c);
    delete c;
}

TgbmBooster *tgbm_booster_create(int n_rows, const float *val, const int *row_ptr, const int *col, const float *label,
                                 const int *group, int num_group, const TgbmParam *param, TgbmComm *comm) {
    TgbmBooster *h = nullptr;
    guard([&] {
        const bool timing = getenv("TGBM_TIMING") != nullptr;  // phase times of the set-up on stderr
        auto t_mark = std::chrono::steady_clock::now();
        auto lap = [&](const char *what) {
            if (!timing) return;
            const auto t = std::chrono::steady_clock::now();
            fprintf(stderr, "[tgbm create] %-26s %8.1f ms\n", what, std::chrono::duration<double, std::milli>(t - t_mark).count());
            t_mark = t;
        };
        std::unique_ptr<TgbmBooster> b(new TgbmBooster);
        b->param = param_from_c(param);
        tgbm::set_verbosity(param->verbose);
        const tgbm::Comm *c = comm ? comm->c : nullptr;
        tgbm::DataSet ds;
        if (c && c->active() && tgbm::need_group_label(tgbm::objective_from_name(b->param.objective))) {
            tgbm::GBMParam tmp = b->param;
            tmp.objective = "reg:linear";  // load without the per-rank label grouping
            ds.load_from_sparse(n_rows, val, row_ptr, col, label, group, num_group, tmp, /*lazy=*/true);
            TGBM_CHECK(label != nullptr, "this objective needs labels");
            group_label_global(ds, label, b->param, c);
        } else {
            ds.load_from_sparse(n_rows, val, row_ptr, col, label, group, num_group, b->param, /*lazy=*/true);
        }
        lap("host view of the data");
        b->label = ds.label;
        b->n_rows = n_rows;
        b->b = new tgbm::Booster(b->param, c);
        b->b->set_profile(param->profile != 0);
        lap("booster object");
        b->b->init(ds);
        lap("init");
        h = b.release();
    });
    return h;
}

int tgbm_booster_boost(TgbmBooster *b, int n_rounds) { return guard([&] { b->b->boost(n_rounds); }); }
int tgbm_booster_sync(TgbmBooster *b) { return guard([&] { b->b->sync(); }); }
int tgbm_booster_set_profile(TgbmBooster *b, int on) { return guard([&] { b->b->set_profile(on != 0); }); }
int tgbm_booster_boost_timed(TgbmBooster *b, int n_rounds, float *elapsed_ms) {
    return guard([&] {
        cudaEvent_t e0, e1;
        TGBM_CUDA(cudaEventCreate(&e0));
        TGBM_CUDA(cudaEventCreate(&e1));
        b->b->sync();
        TGBM_CUDA(cudaEventRecord(e0, b->b->stream()));
        b->b->boost(n_rounds);
        TGBM_CUDA(cudaEventRecord(e1, b->b->stream()));
        b->b->sync();
        TGBM_CUDA(cudaEventElapsedTime(elapsed_ms, e0, e1));
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    });
}
int tgbm_booster_info(TgbmBooster *b, TgbmInfo *o) {
    return guard([&] {
        o->n_rows = b->n_rows; o->n_features = b->b->n_features(); o->fpad = b->b->fpad(); o->n_bins = b->b->n_bins();
        o->trees_per_round = b->b->trees_per_round(); o->n_nodes = b->b->n_nodes(); o->num_class = b->b->num_class();
        o->rounds_done = b->b->rounds_done(); o->n_labels = (int)b->label.size(); o->base_score = b->b->base_score();
        o->csr_layout = b->b->is_sparse() ? 1 : 0;
    });
}
int tgbm_booster_profile(TgbmBooster *b, TgbmProfile *o) {
    return guard([&] {
        const tgbm::HistProfile p = b->b->profile();
        o->hist_ms = p.hist_ms; o->hist_bytes = p.hist_bytes; o->hist_root_ms = p.hist_root_ms; o->hist_root_bytes = p.hist_root_bytes;
        o->partition_ms = p.partition_ms; o->partition_bytes = p.partition_bytes; o->hist_launches = p.hist_launches;
        o->hist_root_launches = p.hist_root_launches; o->partition_launches = p.partition_launches; o->kernel_launches = p.kernel_launches;
        o->hist_rows = p.hist_rows;
    });
}
int tgbm_booster_get_trees(TgbmBooster *b, void *out) {
    return guard([&] {
        auto m = b->b->get_model();
        char *dst = (char *)out;
        for (auto &r : m) for (auto &t : r) { memcpy(dst, t.nodes.data(), sizeof(tgbm::TreeNode) * t.nodes.size()); dst += sizeof(tgbm::TreeNode) * t.nodes.size(); }
    });
}
int tgbm_booster_get_metrics(TgbmBooster *b, float *out) { return guard([&] { auto v = b->b->get_metrics(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_ypred(TgbmBooster *b, float *out) { return guard([&] { auto v = b->b->get_ypred(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_cuts(TgbmBooster *b, float *cut_val, int *cut_ptr) {
    return guard([&] {
        auto v = b->b->get_cut_val(); auto p = b->b->get_cut_ptr();
        std::copy(v.begin(), v.end(), cut_val); std::copy(p.begin(), p.end(), cut_ptr);
    });
}
int tgbm_booster_get_bins(TgbmBooster *b, unsigned char *out) { return guard([&] { auto v = b->b->get_bins(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_bins_csr(TgbmBooster *b, int *out) { return guard([&] { auto v = b->b->get_bins_csr(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_nid(TgbmBooster *b, int *out) { return guard([&] { auto v = b->b->get_nid(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_root_hist(TgbmBooster *b, long long *out) { return guard([&] { auto v = b->b->get_root_hist(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_root_hist_f32(TgbmBooster *b, float *out) { return guard([&] { auto v = b->b->get_root_hist_f32(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_quant_scale(TgbmBooster *b, double *out) { return guard([&] { auto v = b->b->get_quant_scale(); std::copy(v.begin(), v.end(), out); }); }
int tgbm_booster_get_labels(TgbmBooster *b, float *out) { return guard([&] { std::copy(b->label.begin(), b->label.end(), out); }); }
int tgbm_booster_to_model(TgbmBooster *b, ::Tree **model) { return guard([&] { *model = unwrap_model(b->b->get_model()); }); }
void tgbm_booster_free(TgbmBooster *b) {
    delete b;
    tgbm::dev_trim();
}
void tgbm_release_device_memory(void) { tgbm::dev_release_all(); }

int tgbm_metric_score(const char *objective, int n_rows, int trees_per_round, const float *label, const float *raw,
                      const int *group, int num_group, float *out) {
    return guard([&] {
        const int o = tgbm::objective_from_name(objective ? objective : "");
        TGBM_CHECK(o != tgbm::OBJ_UNKNOWN, std::string("undefined objective ") + (objective ? objective : "(null)"));
        TGBM_CHECK(n_rows > 0 && trees_per_round >= 1 && label && raw && out, "bad arguments");
        tgbm::DataSet ds;
        ds.n_rows = n_rows;
        ds.y.assign(label, label + n_rows);
        ds.yv = ds.y.data();
        if (group) ds.group.assign(group, group + num_group);
        std::vector<float> r(raw, raw + (size_t)n_rows * trees_per_round);
        *out = tgbm::metric_score(o, ds, trees_per_round, r);
    });
}

int tgbm_predict_raw(int n_rows, const float *val, const int *row_ptr, const int *col, const void *nodes, int n_rounds,
                     int trees_per_round, int n_nodes, float learning_rate, float base_score, float *out) {
    return tgbm_predict_raw_timed(n_rows, val, row_ptr, col, nodes, n_rounds, trees_per_round, n_nodes, learning_rate, base_score, out,
                                  nullptr);
}

int tgbm_predict_raw_timed(int n_rows, const float *val, const int *row_ptr, const int *col, const void *nodes, int n_rounds,
                           int trees_per_round, int n_nodes, float learning_rate, float base_score, float *out, float *kernel_ms) {
    return guard([&] {
        tgbm::GBMParam p;
        tgbm::DataSet ds;
        ds.load_from_sparse(n_rows, val, row_ptr, col, nullptr, nullptr, 0, p);
        const tgbm::TreeNode *src = (const tgbm::TreeNode *)nodes;
        std::vector<std::vector<tgbm::Tree>> m(n_rounds);
        for (int r = 0; r < n_rounds; ++r) {
            m[r].resize(trees_per_round);
            for (int t = 0; t < trees_per_round; ++t) {
                const tgbm::TreeNode *s = src + ((size_t)r * trees_per_round + t) * n_nodes;
                m[r][t].nodes.assign(s, s + n_nodes);
            }
        }
        std::vector<float> y;
        tgbm::predict_raw(ds, m, learning_rate, base_score, y, kernel_ms);
        std::copy(y.begin(), y.end(), out);
    });
}

}  // extern "C"
