/*
 * C ABI of libthundergbm.so (B200 / sm_100a build of the histogram tree-building path).
 *
 * Part 1 is the reference's own `extern "C"` surface: the functions its Python wrapper binds
 * through ctypes (python/thundergbm/thundergbm.py) and its R wrapper through .C (R/gbm.R).
 * Names, argument order and argument meaning are the reference's.  Where the reference declares
 * `Tree *&model` the ABI is a pointer to the handle, written `Tree **` here.
 *
 * Part 2 is an explicit-state interface to the same path (create / boost / read back) used by the
 * benchmark, by multi-GPU launches (one process per GPU) and by the parity tests.
 *
 * Every entry point works on plain pointers and sizes; all device memory is owned by the library.
 * Functions of part 1 return void like the reference; on failure they log the message, leave
 * `*model` NULL (the Python wrapper tests for that) and keep it for tgbm_last_error().
 */
#ifndef THUNDERGBM_B200_H
#define THUNDERGBM_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct Tree Tree; /* opaque: one tree = 2^(depth+1)-1 node records of 48 bytes */

/* ---------------------------------------------------------------- part 1: reference surface */

/* src/thundergbm/scikit_tgbm.cpp:13-23 -- 0 silent, 1 info, 2 debug */
void set_logger(int verbose);

/* src/thundergbm/scikit_tgbm.cpp:26-80.  CSR is borrowed (copied inside); `col_ptr` is the column
 * index array.  Out: *model = new Tree[n_trees * *tree_per_iter] (free with model_free), *num_class,
 * *tree_per_iter, group_label[0..n_labels). */
void sparse_train_scikit(int row_size, float *val, int *row_ptr, int *col_ptr, float *label, int depth, int n_trees,
                         int n_device, float min_child_weight, float lambda, float gamma, int max_num_bin, int verbose,
                         float column_sampling_rate, int bagging, int n_parallel_trees, float learning_rate,
                         char *obj_type, int *num_class, char *tree_method, Tree **model, int *tree_per_iter,
                         float *group_label, int *group, int num_group);

/* src/thundergbm/scikit_tgbm.cpp:83-121.  y_pred: row_size floats (row_size*num_class, class-major, for
 * multi:softprob), after the objective's predict_transform.  base_score is not applied on this path. */
void sparse_predict_scikit(int row_size, float *val, int *row_ptr, int *col_ptr, float *y_pred, Tree **model,
                           int n_trees, int trees_per_iter, char *objective, int num_class, float learning_rate,
                           float *group_label, int *group, int num_group, int verbose);

/* src/thundergbm/scikit_tgbm.cpp:123-146 -- writes the reference's binary model file (src/thundergbm/parser.cpp:146-171) */
void save(char *model_path, char *objective, float learning_rate, int num_class, int n_trees, int trees_per_iter,
          Tree **model, float *group_label);
/* src/thundergbm/scikit_tgbm.cpp:148-171 */
void load_model(char *model_path, float *learning_rate, int *num_class, int *n_trees, int *trees_per_iter, Tree **model);
/* src/thundergbm/scikit_tgbm.cpp:173-182 */
void load_config(char *model_path, float *group_label);
/* src/thundergbm/scikit_tgbm.cpp:184-197 */
void get_n_nodes(Tree **model, int *n_nodes, int n_trees, int tree_per_iter);
/* src/thundergbm/scikit_tgbm.cpp:199-248 */
void get_a_tree(Tree **model, int tree_id, int n_nodes, int *children_left, int *children_right, int *children_default,
                int *features, float *thresholds, float *values, float *node_sample_weights);
/* src/thundergbm/scikit_tgbm.cpp:250-254 */
void model_free(Tree **model);

/* src/thundergbm/gbm_R_interface.cpp:10-61 and :63-87 (.C calling convention: every argument a pointer) */
void train_R(int *depth, int *n_trees, int *n_gpus, int *verbose, int *profiling, char **data, int *max_num_bin,
             double *column_sampling_rate, int *bagging, int *n_parallel_trees, double *learning_rate, char **objective,
             int *num_class, int *min_child_weight, double *lambda_tgbm, double *gamma, char **tree_method,
             char **model_out);
void predict_R(char **data, char **model_in, int *verbose);

/* ---------------------------------------------------------------- part 2: explicit-state interface */

typedef struct TgbmBooster TgbmBooster;
typedef struct TgbmComm TgbmComm;

typedef struct {
    int depth, n_trees, max_num_bin, num_class;
    float min_child_weight, lambda, gamma, learning_rate;
    const char *objective;
    int quant_bits;     /* value bits of the fixed-point gradient grid (default 18) */
    int keep_nid;       /* keep the final node id of every row for every tree (tests) */
    int verbose;
    int profile;        /* time the histogram and partition kernels with CUDA events */
    unsigned rank_seed; /* LambdaRank partner sampling */
    int hist_mode;      /* histogram arithmetic: 0 fp32 -- float (g,h) added value by value into one accumulator per bin,
                           what the reference does (hist_tree_builder_single.cu:203-216, :485-505); 1 exact -- integer sums
                           on a fixed-point grid, bit-identical from run to run and for any number of GPUs */
    int bagging;        /* RowSampler::do_bagging (src/thundergbm/row_sampler.cu:9-35): bootstrap multiplicities on (g,h) */
    float column_sampling_rate; /* Shard::column_sampling (src/thundergbm/builder/shard.cu:8-23); 1 = off */
    unsigned sample_seed;       /* seed of both samplers (the reference draws from std::rand()) */
    int column_shards;  /* 0: cut points, candidate order and child sums of HistTreeBuilder_single, the reference's builder
                           for n_device = 1; D >= 1: those of the column-sharded HistTreeBuilder it runs for n_device = D > 1
                           (src/thundergbm/builder/hist_tree_builder.cu, hist_cut.cu:104-187), whose cut points depend on D */
    int exact_builder;  /* 1: tree_method = exact, the reference's ExactTreeBuilder (src/thundergbm/builder/exact_tree_builder.cu):
                           every distinct stored value of a node is a split candidate; one GPU */
} TgbmParam;

typedef struct {
    int n_rows, n_features, fpad, n_bins, trees_per_round, n_nodes, num_class, rounds_done, n_labels;
    float base_score;
    int csr_layout; /* 1: wide sparse data kept as CSR of global bin ids, 0: dense byte matrices */
} TgbmInfo;

typedef struct {
    double hist_ms, hist_bytes, hist_root_ms, hist_root_bytes, partition_ms, partition_bytes;
    long long hist_launches, hist_root_launches, partition_launches, kernel_launches;
    long long hist_rows; /* rows the timed histogram launches processed */
} TgbmProfile;

/* message of the last failure on this thread ("" if none) */
const char *tgbm_last_error(void);
void tgbm_default_param(TgbmParam *p);

/* one process per GPU: rank 0 makes the id, every rank calls create with it (NCCL underneath) */
int tgbm_comm_unique_id(unsigned char id[128]);
TgbmComm *tgbm_comm_create(const unsigned char id[128], int rank, int world);
void tgbm_comm_destroy(TgbmComm *c);

/* Booster::init (include/thundergbm/booster.h:36-74): CSR rows of THIS rank -> cut points, bin matrix, base score.
 * `comm` may be NULL.  Returns NULL on failure. */
TgbmBooster *tgbm_booster_create(int n_rows, const float *val, const int *row_ptr, const int *col, const float *label,
                                 const int *group, int num_group, const TgbmParam *param, TgbmComm *comm);
/* Booster::boost x n_rounds; queues the work on the booster's stream and returns */
int tgbm_booster_boost(TgbmBooster *b, int n_rounds);
int tgbm_booster_sync(TgbmBooster *b);
/* boost + sync, bracketed by CUDA events on the booster's stream: device time of the n_rounds in ms */
int tgbm_booster_boost_timed(TgbmBooster *b, int n_rounds, float *elapsed_ms);
/* switch the per-kernel CUDA-event timing of the histogram and partition kernels on or off */
int tgbm_booster_set_profile(TgbmBooster *b, int on);
int tgbm_booster_info(TgbmBooster *b, TgbmInfo *out);
int tgbm_booster_profile(TgbmBooster *b, TgbmProfile *out);
/* rounds_done * trees_per_round * n_nodes records of 48 bytes */
int tgbm_booster_get_trees(TgbmBooster *b, void *nodes_out);
int tgbm_booster_get_metrics(TgbmBooster *b, float *out);            /* rounds_done */
int tgbm_booster_get_ypred(TgbmBooster *b, float *out);              /* trees_per_round * n_rows */
int tgbm_booster_get_cuts(TgbmBooster *b, float *cut_val, int *cut_ptr); /* n_bins, n_features+1 */
int tgbm_booster_get_bins(TgbmBooster *b, unsigned char *out);       /* dense layout: n_rows * fpad, 255 = missing */
int tgbm_booster_get_bins_csr(TgbmBooster *b, int *out);             /* CSR layout: global bin id per stored value */
int tgbm_booster_get_nid(TgbmBooster *b, int *out);                  /* rounds_done*trees_per_round*n_rows (keep_nid) */
int tgbm_booster_get_root_hist(TgbmBooster *b, long long *out);      /* exact mode: n_bins*2 of the last tree */
int tgbm_booster_get_root_hist_f32(TgbmBooster *b, float *out);      /* fp32 mode: n_bins*2 of the last tree */
int tgbm_booster_get_quant_scale(TgbmBooster *b, double *out);       /* rounds_done*2 */
int tgbm_booster_get_labels(TgbmBooster *b, float *out);             /* n_labels */
/* hands the trained trees over as the opaque model of part 1 */
int tgbm_booster_to_model(TgbmBooster *b, Tree **model);
void tgbm_booster_free(TgbmBooster *b);
/* The library's device buffers come from one memory pool per GPU that keeps what a call releases (up to
 * TGBM_POOL_KEEP_MB megabytes, default 16384; TGBM_NO_POOL=1: plain cudaMalloc / cudaFree), so that the next call finds
 * its memory mapped.  This gives every unused block back to the driver now. */
void tgbm_release_device_memory(void);

/* Predictor::predict_raw (src/thundergbm/predictor.cu:32-189) on node records as returned by
 * tgbm_booster_get_trees: out[t * n_rows + i] */
int tgbm_predict_raw(int n_rows, const float *val, const int *row_ptr, const int *col, const void *nodes, int n_rounds,
                     int trees_per_round, int n_nodes, float learning_rate, float base_score, float *out);
/* the same, also returning the device time of the traversal kernel alone (measurement) */
int tgbm_predict_raw_timed(int n_rows, const float *val, const int *row_ptr, const int *col, const void *nodes, int n_rounds,
                     int trees_per_round, int n_nodes, float learning_rate, float base_score, float *out, float *kernel_ms);

/* Metric::get_score of the objective's default metric (the .cu files under src/thundergbm/metric, rank_metric.cpp) on raw scores
 * raw[t * n_rows + i]: RMSE, binary error, multi-class accuracy, MAP or NDCG.  `label` holds class indices for the
 * classification objectives.  Host pointers; device buffers and reduction scratch are allocated inside. */
int tgbm_metric_score(const char *objective, int n_rows, int trees_per_round, const float *label, const float *raw,
                      const int *group, int num_group, float *out);

/* The same metric for callers that must not allocate device memory: a host whose own pool already owns the whole
 * GPU, or a hook inside another program's step loop that cannot afford the device-wide synchronisation of
 * cudaMalloc / cudaFree.  No counterpart in the reference (every reference entry point allocates).
 * d_label, d_raw (raw[t * n_rows + i]) and d_out (one float) are DEVICE pointers owned by the caller; the kernels
 * are queued on `cuda_stream` (a cudaStream_t, NULL = default stream) and the call returns without waiting.
 * The reduction scratch is a fixed 8.2 KB array inside the library image on every GPU that loads the library.
 * n_rows <= TGBM_NOALLOC_MAX_ROWS, trees_per_round <= TGBM_NOALLOC_MAX_CLASSES, no ranking objectives; anything else
 * returns 1 with the reason in tgbm_last_error().  The first call on each device resolves the scratch address and
 * should be made outside stream capture.  All calls on a device share the scratch: calls whose kernels can overlap
 * on the GPU (unordered streams) race; calls on one stream are safe. */
#define TGBM_NOALLOC_MAX_ROWS (1 << 30)
#define TGBM_NOALLOC_MAX_CLASSES 1024
int tgbm_metric_score_noalloc(const char *objective, int n_rows, int trees_per_round, const float *d_label,
                              const float *d_raw, float *d_out, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
