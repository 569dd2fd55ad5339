// Shared host-side types of the B200 histogram tree builder.
#pragma once
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

namespace tgbm {

// 48-byte node record; byte-compatible with the reference's Tree::TreeNode
// (include/thundergbm/tree.h:14-42), which is also the model-file record
// (src/thundergbm/parser.cpp:146-171).
struct TreeNode {
    int final_id, lch_index, rch_index, parent_index;
    float gain, base_weight;
    int split_feature_id;
    float split_value;
    unsigned char split_bid;
    unsigned char default_right, is_leaf, is_valid, is_pruned;  // bools in the reference
    unsigned char pad_[3];
    float sum_g, sum_h;
};
static_assert(sizeof(TreeNode) == 48, "TreeNode must stay 48 bytes");

// The opaque `Tree` of the C API (src/thundergbm/scikit_tgbm.cpp): one node table per tree.
struct Tree {
    std::vector<TreeNode> nodes;
};

enum Objective { REG_LINEAR = 0, REG_LOGISTIC = 1, BINARY_LOGISTIC = 2, MULTI_SOFTMAX = 3, MULTI_SOFTPROB = 4,
                 RANK_PAIRWISE = 5, RANK_NDCG = 6, OBJ_UNKNOWN = -1 };

inline int objective_from_name(const std::string &s) {  // src/thundergbm/objective/objective_function.cu:9-19
    if (s == "reg:linear") return REG_LINEAR;
    if (s == "reg:logistic") return REG_LOGISTIC;
    if (s == "binary:logistic") return BINARY_LOGISTIC;
    if (s == "multi:softprob") return MULTI_SOFTPROB;
    if (s == "multi:softmax") return MULTI_SOFTMAX;
    if (s == "rank:pairwise") return RANK_PAIRWISE;
    if (s == "rank:ndcg") return RANK_NDCG;
    return OBJ_UNKNOWN;
}
inline bool need_group_label(int o) { return o == MULTI_SOFTPROB || o == MULTI_SOFTMAX || o == BINARY_LOGISTIC; }
inline bool need_group_file(int o) { return o == RANK_PAIRWISE || o == RANK_NDCG; }
inline const char *metric_name(int o) {  // default_metric_name() + Metric::get_name() of the reference
    switch (o) {
    case REG_LINEAR: case REG_LOGISTIC: return "RMSE";
    case BINARY_LOGISTIC: return "test error";
    case MULTI_SOFTMAX: case MULTI_SOFTPROB: return "multi-class accuracy";
    case RANK_PAIRWISE: return "MAP";
    case RANK_NDCG: return "NDCG";
    }
    return "?";
}

// include/thundergbm/common.h:86-111 (same fields, same defaults as src/thundergbm/parser.cpp:10-28)
struct GBMParam {
    int depth = 6;
    int n_trees = 40;
    float min_child_weight = 1;
    float lambda = 1;
    float gamma = 1;
    float rt_eps = 1e-6f;
    float column_sampling_rate = 1;
    std::string path = "../dataset/test_dataset.txt";
    int verbose = 1;
    bool profiling = false;
    bool bagging = false;
    int n_parallel_trees = 1;
    float learning_rate = 1;
    std::string objective = "reg:linear";
    int num_class = 1;
    int tree_per_rounds = 1;
    int max_num_bin = 255;
    float base_score = 0;
    int n_device = 1;
    std::string tree_method = "auto";
    // additions of this implementation
    // Histogram arithmetic.  0 "fp32": float (g,h) added per stored value into one accumulator per bin, float prefix
    // sums -- the reference's own arithmetic (hist_tree_builder_single.cu:203-216), results depend on the order of
    // the additions in the last bits.  1 "exact": gradients on a power-of-two grid, integer sums -- the deterministic
    // mode: bit-identical from run to run and for any number of GPUs.
    int hist_mode = 0;
    // 0: cut points, candidate order and child sums of the one-device builder (HistTreeBuilder_single, what the
    // reference runs for n_device = 1).  D >= 1: those of the column-sharded HistTreeBuilder the reference runs for
    // n_device = D > 1 -- its cut points depend on D (each device shifts and re-rounds the values of its own block
    // of columns, hist_cut.cu:104-134).  The rows are still sharded over this implementation's own GPUs.
    int column_shards = 0;
    int quant_bits = 18;        // exact mode: value bits of the fixed-point gradient grid
    unsigned sample_seed = 0;   // bagging and column sampling (the reference draws from std::rand())
    unsigned rank_seed = 0;     // LambdaRank partner sampling
    int keep_nid = 0;           // tests: keep ins2node_id of every tree
};

// "fp32" / "0" and "exact" / "deterministic" / "1"; anything else is -1 (rejected by Booster::init)
inline int hist_mode_from_name(const std::string &s) {
    if (s == "fp32" || s == "0") return 0;
    if (s == "exact" || s == "deterministic" || s == "1") return 1;
    return -1;
}
// Default histogram arithmetic of the entry points whose signature has no room for it (the reference's own C
// surface): the environment variable TGBM_HIST_MODE, else fp32.
int default_hist_mode();

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

#define TGBM_CHECK(cond, msg)                                                              \
    do {                                                                                   \
        if (!(cond)) throw ::tgbm::Error(std::string(msg) + " (" #cond ") at " __FILE__ ":" + std::to_string(__LINE__)); \
    } while (0)

// host data set: CSR + labels (src/thundergbm/dataset.cpp)
struct DataSet {
    int n_rows = 0;
    int n_features = 0;
    // CSR views: borrowed from the caller (load_from_sparse; valid for the duration of the call, like the
    // reference's copies) or pointing into the owned vectors below (load_from_file)
    const int *rp = nullptr, *ci = nullptr;
    const float *vv = nullptr;
    std::vector<int> row_ptr, col;
    std::vector<float> val, y;
    std::vector<int> group;
    std::vector<float> label;  // distinct class labels after group_label()
    // Labels as the booster reads them: `y` (owned) or the caller's array (borrowed).  labels_raw: the objective
    // groups its labels (dataset.cpp:83-101) but `yv` still holds the caller's values -- `label` is complete and the
    // booster maps y -> index on the device.
    const float *yv = nullptr;
    bool labels_raw = false;
    // lazy = true does on the host only what needs no pass that writes: n_features stays -1 (the booster finds it on
    // the device after the upload) and the labels are borrowed instead of copied.
    void load_from_sparse(int n, const float *v, const int *rp, const int *ci, const float *yy, const int *grp,
                          int num_group, GBMParam &param, bool lazy = false);
    void distinct_labels(const float *yy, size_t n);
    int count_features() const;   // largest column index + 1, scanned by a few host threads
    void load_from_file(const std::string &file, GBMParam &param);
    void load_group_file(const std::string &file);
    void group_label();
};

// logging (verbosity as in set_logger: 0 silent, 1 info, 2 debug)
void set_verbosity(int v);
int verbosity();
void log_info(const char *fmt, ...);

// message returned by tgbm_last_error() on the calling thread
void set_last_error(const std::string &msg);

void parse_param(GBMParam &p, int argc, char **argv);
void save_model(const std::string &path, const GBMParam &p, const std::vector<std::vector<Tree>> &model,
                const std::vector<float> &label);
void load_model(const std::string &path, GBMParam &p, std::vector<std::vector<Tree>> &model, std::vector<float> &label);

}  // namespace tgbm
