// Booster: the boosting loop and the per-level tree builder on one GPU (one rank).
// Counterpart of Booster / TreeBuilder::build_approximate / HistTreeBuilder_single in the reference
// (include/thundergbm/booster.h:36-93, src/thundergbm/builder/tree_builder.cu:147-194,
// src/thundergbm/builder/hist_tree_builder_single.cu).
#pragma once
#include <cuda_runtime.h>

#include <memory>
#include <vector>

#include "tgbm_comm.h"
#include "tgbm_common.h"

namespace tgbm {

struct BoosterImpl;

struct HistProfile {
    double hist_ms = 0;          // summed device time of the histogram-build kernels
    long long hist_launches = 0;
    double hist_bytes = 0;       // algorithmic bytes they processed
    double partition_ms = 0;
    long long partition_launches = 0;
    double partition_bytes = 0;
    long long kernel_launches = 0;  // every kernel of this library launched by boost()
    double hist_root_ms = 0;
    double hist_root_bytes = 0;
    long long hist_root_launches = 0;
    long long hist_rows = 0;       // rows those histogram launches processed (root + gathered)
};

class Booster {
public:
    // `comm` may be null (single GPU).  The booster keeps the pointer, the caller owns it.
    Booster(const GBMParam &param, const Comm *comm);
    ~Booster();

    // Host CSR -> device, cut points, bin matrix, labels, base score.  With a communicator each rank passes its
    // own contiguous block of rows; n_features must then be the global feature count.
    void init(const DataSet &ds);
    // rounds [done, done+n) ; asynchronous on the booster's stream
    void boost(int n_rounds);
    void sync();

    int rounds_done() const;
    int trees_per_round() const;
    int n_nodes() const;
    int num_class() const;
    float base_score() const;
    int n_bins() const;
    int n_features() const;
    std::string tree_method() const;   // after init(): "hist" or "exact" (auto resolved)
    int fpad() const;
    cudaStream_t stream() const;
    void set_profile(bool on);
    HistProfile profile();  // syncs

    std::vector<std::vector<Tree>> get_model();           // syncs
    std::vector<float> get_metrics();                     // per finished round; syncs
    std::vector<float> get_ypred();                       // [K][N] raw scores of the training rows
    std::vector<float> get_cut_val() const;
    std::vector<int> get_cut_ptr() const;
    std::vector<unsigned char> get_bins();                // dense layout: [N][Fpad] local bin ids, 255 = missing
    std::vector<int> get_bins_csr();                      // CSR layout: global bin id per stored value
    bool is_sparse() const;
    std::vector<int> get_nid();                           // [tree][N] when param.keep_nid
    std::vector<long long> get_root_hist();               // exact mode: [B][2] level-0 histogram of the last tree built
    std::vector<float> get_root_hist_f32();               // fp32 mode: the same as float pairs
    std::vector<double> get_quant_scale();                // per round: scale_g, scale_h

private:
    std::unique_ptr<BoosterImpl> impl_;
};

// TreeTrainer::train (src/thundergbm/trainer.cu:18-57) for the histogram path: one booster on the current device, or --
// param.n_device > 1 -- one host thread per GPU on devices 0 .. n_device-1 with the rows sharded between them.
// Logs the per-round metric and the training time like the reference; updates base_score, num_class, tree_per_rounds.
std::vector<std::vector<Tree>> train_model(GBMParam &param, const DataSet &ds);

// batch inference, Predictor::predict_raw (src/thundergbm/predictor.cu:32-189): out[t*N+i]
// kernel_ms (optional): device time of the traversal kernel alone
void predict_raw(const DataSet &ds, const std::vector<std::vector<Tree>> &model, float learning_rate, float base_score,
                 std::vector<float> &out, float *kernel_ms = nullptr);
// ObjectiveFunction::predict_transform on raw scores (in place; may shrink `y`)
void predict_transform(int objective, int num_class, const std::vector<float> &label, int n_rows, std::vector<float> &y);
// Metric::get_score on raw scores of `ds`
float metric_score(int objective, const DataSet &ds, int num_class, const std::vector<float> &raw);

}  // namespace tgbm
