// Host class of the hash-grid network (multiresolution hash encoding + fused MLP), source-compatible with the
// reference's TinyMLPHashGrid (modules/TinyMLP/TinyMLPHashGrid.h:11-85).  Parameters live in one arena slice
// [hash table L*T*2 | weights | biases]; the level geometry is computed once at construction.
#pragma once

#include "TinyMLP.h"

// Field order is part of the weight-file format (modules/TinyMLP/TinyMLPHashGrid.h:11-23).
struct MLPGridOptions {
    int vectorDim;  // 3 or 4 floats per input point
    int hiddenDim;
    int outputDim;
    int numLayers;
    int activationType;

    int tableSize;
    int numLevels;
    float b;
    int lowestSize;
    int featuresLevel;  // must be 2
};

inline int inputDim(MLPGridOptions& opt) { return opt.featuresLevel * opt.numLevels; }

class TinyMLPHashGrid {
public:
    explicit TinyMLPHashGrid(const MLPGridOptions& options, int maxBatchSize, int inferBatchSize = 0, unsigned int seed = 42,
                             bool isTraining = true);
    // Places hash table, weights and biases inside an existing arena: the table at hash_offset, the network at
    // mlp_offset.  The arena must outlive the object.  No counterpart in the reference.
    TinyMLPHashGrid(const MLPGridOptions& options, int maxBatchSize, int inferBatchSize, unsigned int seed, bool isTraining,
                    nb::ParamArena* arena, int64_t hash_offset, int64_t mlp_offset);
    ~TinyMLPHashGrid();
    TinyMLPHashGrid(const TinyMLPHashGrid&) = delete;
    TinyMLPHashGrid& operator=(const TinyMLPHashGrid&) = delete;

    void switchToInferenceMode();
    void switchToTrainingMode();

    void zero_grad(cudaStream_t stream = 0);
    void forward(const float* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream = 0);
    float calculate_loss_and_grad(const half* d_unpadded_targets, int batchSize, float loss_scale = 65536.0f, bool fetch_loss = false,
                                  cudaStream_t stream = 0);
    void backward(int batchSize, cudaStream_t stream = 0);
    void backward(const half* custom_loss_grad, int batchSize, cudaStream_t stream = 0);

    // Kept for source compatibility: the scatter always runs as its own per-level kernel here.
    void setSplitScatter(bool enabled) { m_useSplitScatter = enabled; }
    bool getSplitScatter() const { return m_useSplitScatter; }

    void step(float lr = 3e-4f, float beta1 = 0.9f, float beta2 = 0.999f, float epsilon = 1e-8f, float loss_scale = 65536.0f,
              cudaStream_t stream = 0);
    void reset_step();
    void inference(const float* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream = 0);

    void loadWeights(const std::string& filename);
    void saveWeights(const std::string& filename);
    void loadWeights(const float* host_weights, const float* host_biases);
    void saveWeights(float* host_weights, float* host_biases);
    void loadHashgrid(const float* host_hashgrid);
    void saveHashgrid(float* host_hashgrid);

    // ---- additions (not in the reference) -------------------------------------------------------------
    static int64_t hashCount(const MLPGridOptions& options) { return (int64_t)options.numLevels * options.tableSize * options.featuresLevel; }
    static int64_t mlpParamCount(const MLPGridOptions& options);
    const nb_grid_desc& grid() const { return grid_; }
    const nb_mlp_desc& desc() const { return desc_; }
    int64_t hashOffset() const { return off_hash_; }
    int64_t weightOffset() const { return off_w_; }
    int64_t biasOffset() const { return off_b_; }
    int64_t weightCount() const { return n_w_; }
    int64_t biasCount() const { return n_b_; }
    half* encodedInput() const { return enc_.as<half>(); }
    half* hiddenActivations() const { return acts_.as<half>(); }
    half* encodingGradient() const { return denc_.as<half>(); }
    float* paddedOutput() const { return padded_out_.as<float>(); }

private:
    void construct(unsigned int seed, nb::ParamArena* arena, int64_t hash_offset, int64_t mlp_offset);
    void allocate_buffers();
    void run_backward(const half* grad_padded, int batchSize, cudaStream_t stream);

    MLPGridOptions user_opt;
    MLPGridOptions hw_opt;
    MLPOption mlp_opt;
    nb_grid_desc grid_{};
    nb_mlp_desc desc_{};
    int m_maxBatchSize;
    int m_inferBatchSize;
    int current_step = 0;
    bool m_isTraining;
    bool m_useSplitScatter = true;

    std::unique_ptr<nb::ParamArena> owned_;
    nb::ParamArena* arena_ = nullptr;
    int64_t off_hash_ = 0, off_w_ = 0, off_b_ = 0, n_hash_ = 0, n_w_ = 0, n_b_ = 0;

    const float* last_inputs_ = nullptr;  // float4 positions of the last forward (caller's buffer when vectorDim == 4)
    nb::DeviceMem padded_in_, padded_targets_, padded_out_, dloss_, total_loss_, enc_, acts_, denc_;
};
