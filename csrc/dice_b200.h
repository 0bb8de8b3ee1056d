// C interface of libdice_b200 (sm_100a).  All pointers are device pointers unless stated otherwise; `stream` is a
// cudaStream_t passed as void*.  Functions return 0 when the launch was accepted; device-side failures (bounded
// waits that gave up, bad indices) are reported through the caller-provided status word.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest batch (number of data points) the allocation-free entry point accepts.
#define DICE_NOALLOC_MAX_BATCH 65536

int dice_positive_scan(const long long* dp_idx, const long long* offsets, int n, int* first, void* stream);

int dice_positive_correction(const long long* dp_idx, const long long* offsets, const long long* values,
                             const int* first, const void* q, const void* e, float* dq, float* de, double* loss,
                             float weight, float scale, int n, int D, int W, int rank, float* const* dq_table,
                             int dq_block_rows, void* stream);

// Allocation-free variant of dice_positive_scan + dice_positive_correction.  This entry point has no counterpart in
// the reference implementation (which has no native code at all); it exists for callers that cannot allocate
// device memory: the int[n + 1] prefix-sum scratch lives in a fixed __device__ array inside the library
// (DICE_NOALLOC_MAX_BATCH + 1 ints per GPU that loads the library).  n > DICE_NOALLOC_MAX_BATCH returns -7.
// The first call on a device resolves the array's device address and should happen before any stream capture.
// Calls share the array: calls that overlap on the GPU race and must be serialised by the caller.
int dice_positive_correction_noalloc(const long long* dp_idx, const long long* offsets, const long long* values,
                                     const void* q, const void* e, float* dq, float* de, double* loss, float weight,
                                     float scale, int n, int D, int W, int rank, void* stream);

// Convolutional gate (3x3 convolution with one input channel, batch normalisation, ReLU) of the ConEx / ConvQ /
// ConvO model families.  dice_conv_gate_supported returns 1 when the shape is covered.
int dice_conv_gate_supported(int B, int H, int W, int C);
int dice_conv_gate_forward(int B, int H, int W, int C, int training, const float* X, const float* w,
                           const float* bias, const float* gamma, const float* beta, float* run_mean, float* run_var,
                           float momentum, float eps, double* stats, float* fold, float* F, void* stream);
int dice_conv_gate_backward(int B, int H, int W, int C, int training, const float* X, const float* w,
                            const float* bias, const float* fold, const float* dF, double* bstats, float* dX,
                            double* dwb, void* stream);

#ifdef __cplusplus
}
#endif
