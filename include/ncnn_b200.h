/*
 * ncnn_b200.h -- C ABI of the B200 (sm_100a) inference runtime that stands in for
 * the shared library emitted by hqu-little-boy/ncnn-compiler's `ncnn-compile`.
 *
 * The reference product exports, per compiled model, one function
 *     int <model>(const float *input1, ..., float *output1, ...)
 * (tools/ncnn-compile.cpp:1108-1162; wrapper built by lib/Transforms/GenerateCAPI/
 * GenerateCAPI.cpp:975-1090) with status codes 0..5 (tools/ncnn-compile.cpp:955-960),
 * caller-owned contiguous fp32 [C][H][W] buffers, and loads `.param`/`.bin` in its
 * front end (lib/Graph/graph.cpp:2129-2333, API include/ncnn-mlir/Graph/graph.hpp:379-380).
 * This header is what an FFI binds instead: plain pointers and sizes, no C++ types,
 * no exceptions across the boundary.  There is no CPU path: every entry point that
 * computes needs a B200 and fails with NCNN_B200_STATUS_RUNTIME otherwise.
 */
#ifndef NCNN_B200_H_
#define NCNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  0..5 keep the meaning of the reference's generated header
 * (tools/ncnn-compile.cpp:955-960); 6.. are additions of this runtime. */
#define NCNN_B200_STATUS_SUCCESS 0
#define NCNN_B200_STATUS_NULL_POINTER 1
#define NCNN_B200_STATUS_INVALID_SHAPE 2
#define NCNN_B200_STATUS_CONSTRAINT_VIOLATION 3
#define NCNN_B200_STATUS_SHAPE_OVERFLOW 4
#define NCNN_B200_STATUS_OUTPUT_CAPACITY 5
#define NCNN_B200_STATUS_RUNTIME 6  /* CUDA error, out of memory, no device */
#define NCNN_B200_STATUS_TIMEOUT 7  /* a bounded device-side wait gave up */
#define NCNN_B200_STATUS_LOAD 8     /* .param/.bin rejected or layer unsupported */

/* Accuracy modes of fp32 contractions (Convolution, InnerProduct, Gemm). */
#define NCNN_B200_FP32_SPLIT 0 /* tensor cores, split operands (bf16 pairs, else tf32 pairs), 3 MMAs, ~1e-5 relative */
#define NCNN_B200_TF32 1       /* tensor cores, single TF32 pass, ~1e-3 relative     */
#define NCNN_B200_FP32_CUDA 2  /* CUDA-core fp32 FMA                                 */

typedef struct ncnn_b200_model ncnn_b200_model;

typedef struct ncnn_b200_options {
  uint32_t struct_size;   /* sizeof(ncnn_b200_options) */
  int32_t accuracy_mode;  /* NCNN_B200_FP32_SPLIT (default) ... */
  int32_t device;         /* CUDA device ordinal, -1 = current */
  int32_t use_cuda_graph; /* 1 = replay a captured graph per batch size (default) */
  /* Shapes for Input layers that carry no dimensions (the reference takes them from
   * `--input-shape`, tools/ncnn-compile.cpp:40-198), in Input order: for each, the rank
   * followed by that many extents, outermost first ([c,h,w]). */
  int32_t input_shape_count;
  const int64_t *input_shapes;
  /* 1 = parse, validate and infer shapes only, without touching a GPU: enough for
   * ncnn_b200_emit_stub and the shape queries (a compile step), not for running. */
  int32_t plan_only;
  /* 1 = an InnerProduct whose input is a rank-2 [M,K] tensor keeps its rows ([M,N]) also when
   * M is 1, as the reference lowers a dynamic M (NCNNToTosa.cpp:5290-5303); 0 = a static input
   * with exactly K elements is flattened to [N] (NCNNOps.cpp:1247-1312).  Set by the dynamic
   * loader for its specialisations. */
  int32_t keep_matrix_rows;
} ncnn_b200_options;

/* Replaces ncnn_graph::Graph::load + the compile pipeline (graph.hpp:379-380,
 * tools/ncnn-compile.cpp:1824-1888): reads the files, fuses and plans the graph, packs
 * and uploads the weights.  On failure *out is NULL and ncnn_b200_last_error(NULL)
 * describes why. */
int ncnn_b200_load(const char *param_path, const char *bin_path, const ncnn_b200_options *options,
                   ncnn_b200_model **out);
void ncnn_b200_free(ncnn_b200_model *model);

/* Message of the last failure on `model`, or of the last failed load when model is
 * NULL.  The pointer stays valid until the next call on the same model/thread. */
const char *ncnn_b200_last_error(const ncnn_b200_model *model);

/* Argument order follows the reference: Input-layer tops in layer order, then output
 * blobs in creation order (lib/Graph/graph.cpp:2311-2324).  Shapes are per image,
 * outermost first; the return value is the rank (1..3) or -1. */
int ncnn_b200_input_count(const ncnn_b200_model *model);
int ncnn_b200_output_count(const ncnn_b200_model *model);
int ncnn_b200_input_shape(const ncnn_b200_model *model, int index, int64_t dims[3]);
int ncnn_b200_output_shape(const ncnn_b200_model *model, int index, int64_t dims[3]);
/* The same for tensors of rank up to 4 ([c,d,h,w]: the reference's rank-4 Reshape / Permute / Slice / Concat results,
 * lib/Importer/ImportOps.cpp:166-300, ImportTensor.cpp:343-400); the three-extent forms answer -1 for rank 4. */
int ncnn_b200_input_shape4(const ncnn_b200_model *model, int index, int64_t dims[4]);
int ncnn_b200_output_shape4(const ncnn_b200_model *model, int index, int64_t dims[4]);
const char *ncnn_b200_input_name(const ncnn_b200_model *model, int index);
const char *ncnn_b200_output_name(const ncnn_b200_model *model, int index);

/* One image, host buffers: the body of the reference's exported
 * `int <model>(const float *input1, ..., float *output1, ...)`
 * (GenerateCAPI.cpp:1032-1090).  Any NULL pointer returns 1, like the wrapper's
 * null checks (:1053-1077). */
int ncnn_b200_run(ncnn_b200_model *model, const float *const *inputs, float *const *outputs);

/* Extension (the reference has no batch dimension, NCNNToTosa.cpp:48-52): n images
 * back to back per argument; equals n calls of ncnn_b200_run. */
int ncnn_b200_run_batch(ncnn_b200_model *model, int64_t n, const float *const *inputs,
                        float *const *outputs);

/* Same with device pointers on the caller's CUDA stream (a cudaStream_t passed as
 * void*); asynchronous.  ncnn_b200_check_status reports a device-side time-out after
 * the caller synchronised.
 * One call in flight per handle: a model owns one activation arena, so the next call on the
 * same handle (on any stream, including ncnn_b200_launch_count and a run with a batch size
 * not seen before, which lay the arena out anew) belongs after the previous one has finished.
 * The first use of a new batch size synchronises the device for that reason.  Plans (CUDA
 * graphs, staging buffers) are cached for the eight most recently used batch sizes.
 * Every entry point makes the model's device (options.device) current for the call and puts
 * the caller's device back before it returns. */
int ncnn_b200_run_batch_device(ncnn_b200_model *model, int64_t n, const float *const *inputs,
                               float *const *outputs, void *stream);
int ncnn_b200_check_status(ncnn_b200_model *model);

/* Number of kernel launches one run of batch n issues. */
int ncnn_b200_launch_count(ncnn_b200_model *model, int64_t n);

/* Per-launch timing of batch n (CUDA events, `repeat` runs after one warm-up), written
 * as text lines "kernel<TAB>layer<TAB>ms<TAB>flops<TAB>bytes".  Returns the number
 * of bytes needed (excluding the terminator) or a negative status. */
int64_t ncnn_b200_profile(ncnn_b200_model *model, int64_t n, int repeat, char *buffer,
                          size_t capacity);

/* Loader only, no GPU needed: text in the layout of the reference's Graph::dump()
 * (lib/Graph/graph.cpp:2335-2446) plus one FNV-1a hash per weight tensor, or
 * "ERROR: <message>".  Returns the number of bytes needed (excluding the terminator). */
int64_t ncnn_b200_describe(const char *param_path, const char *bin_path, char *buffer,
                           size_t capacity);

/* Writes `<dir>/<name>.h` in the layout of the reference's generated header
 * (tools/ncnn-compile.cpp:945-1218) and `<dir>/<name>.c`, a stub that exports
 * `int <name>(const float *input1, ..., float *output1, ...)`, lazily loads the
 * given .param/.bin through this library and forwards to ncnn_b200_run. */
int ncnn_b200_emit_stub(const ncnn_b200_model *model, const char *name, const char *param_path,
                        const char *bin_path, const char *directory);

/* ---- fixed-rank dynamic input shapes ---------------------------------------------------
 * Replaces the dynamic half of the reference's generated wrapper: models compiled with
 * `--input-shape=3x?x?` / `--input-dim-constraint=0:1:min=32,multiple=32`
 * (docs/ncnn-compile-command-line.md 2.5-2.6) export
 *     int <model>(const float *input1, const int64_t input1_shape[3], float *output1,
 *                 uint64_t output1_capacity)
 *     int <model>_infer_output_shapes(const int64_t input1_shape[3], int64_t output1_shape[R])
 * (tools/ncnn-compile.cpp:1108-1215; test/Numerical/support/numerical_test_support.cpp:204-263),
 * whose wrapper validates in this order (lib/Transforms/GenerateCAPI/GenerateCAPI.cpp:1053-1480):
 * NULL pointer 1; dynamic extent <= 0 or static extent mismatch 2; minimum / multiple violated 3;
 * element or byte count overflow 4; non-positive result extent 2; capacity (elements) too small 5.
 * Here a dynamic model is a table of static specialisations keyed by the extents: the first call
 * with a new shape plans (and for a run, packs and uploads) it, later calls replay it; the 8 most
 * recently used runnable specialisations are kept. */
typedef struct ncnn_b200_dynamic_model ncnn_b200_dynamic_model;

typedef struct ncnn_b200_dim_constraint {
  int32_t input;       /* Input index, layer order */
  int32_t dim;         /* dimension of that input, [c,h,w] order; must be dynamic */
  int64_t minimum;     /* > 0 */
  int64_t multiple_of; /* > 0 */
} ncnn_b200_dim_constraint;

/* `options->input_shapes` holds one template per Input without dimensions, as for
 * ncnn_b200_load, with -1 for every `?` extent.  Needs no GPU (shapes are planned, nothing is
 * uploaded until the first run).  Invalid constraints fail here, as they fail the reference's
 * compile step. */
int ncnn_b200_dynamic_load(const char *param_path, const char *bin_path, const ncnn_b200_options *options,
                           const ncnn_b200_dim_constraint *constraints, int32_t constraint_count,
                           ncnn_b200_dynamic_model **out);
void ncnn_b200_dynamic_free(ncnn_b200_dynamic_model *model);
const char *ncnn_b200_dynamic_last_error(const ncnn_b200_dynamic_model *model);
int ncnn_b200_dynamic_input_count(const ncnn_b200_dynamic_model *model);
int ncnn_b200_dynamic_output_count(const ncnn_b200_dynamic_model *model);
/* Rank and extents, -1 where the extent is dynamic (for outputs: where it follows the inputs). */
int ncnn_b200_dynamic_input_shape(const ncnn_b200_dynamic_model *model, int index, int64_t dims[3]);
int ncnn_b200_dynamic_output_shape(const ncnn_b200_dynamic_model *model, int index, int64_t dims[3]);
/* `input_shapes[i]` is read for inputs with a dynamic extent (others may be NULL);
 * `output_shapes[o]` receives rank-many extents when not NULL. */
int ncnn_b200_dynamic_infer_output_shapes(ncnn_b200_dynamic_model *model, const int64_t *const *input_shapes,
                                          int64_t *const *output_shapes);
/* One image, host buffers.  `output_capacities[o]` (elements) is read for outputs with a
 * dynamic extent. */
int ncnn_b200_dynamic_run(ncnn_b200_dynamic_model *model, const float *const *inputs,
                          const int64_t *const *input_shapes, float *const *outputs,
                          const uint64_t *output_capacities);
/* Header, manifest and stub for the two reference entry points above. */
int ncnn_b200_dynamic_emit_stub(const ncnn_b200_dynamic_model *model, const char *name, const char *param_path,
                                const char *bin_path, const char *directory);

/* Stand-alone int8 boundary operators on device arrays (cudaStream_t as void*).
 * Element i belongs to channel (i / inner) % channels; scale/bias counts are 1 or
 * `channels`.  Replace ConvertQuantize / ConvertDequantize / ConvertRequantize
 * (lib/Conversion/NCNNToTosa/NCNNToTosa.cpp:4802-4888). */
int ncnn_b200_op_quantize(const float *x, int8_t *y, int64_t count, int64_t inner, int32_t channels,
                          const float *scale, int32_t scale_count, void *stream);
int ncnn_b200_op_dequantize(const int32_t *x, float *y, int64_t count, int64_t inner,
                            int32_t channels, const float *scale, int32_t scale_count,
                            const float *bias, int32_t bias_count, void *stream);
int ncnn_b200_op_requantize(const int32_t *x, int8_t *y, int64_t count, int64_t inner,
                            int32_t channels, const float *scale_in, int32_t scale_in_count,
                            const float *scale_out, int32_t scale_out_count, const float *bias,
                            int32_t bias_count, int32_t relu, void *stream);

/* ---- One model on several GPUs of one box (batch sharding).
 * The reference has no counterpart: its entry point takes one image per call and keeps no state between
 * calls (lib/Conversion/NCNNToTosa/NCNNToTosa.cpp:48-52), which is what makes the images of a batch
 * independent.  A multi-device handle keeps one replica of the model per listed device (weights copied to
 * each, one stream, one captured graph and one host thread per device).  ncnn_b200_multi_run_batch cuts the
 * n images into contiguous shards of ceil(n / devices) images (ncnn_b200_multi_partition gives the cut),
 * every device runs its shard, and each copies its results straight into the caller's host arrays: no
 * collective and no peer traffic.  A device ordinal may be listed more than once (two replicas on one GPU).
 * Arguments and status codes are those of ncnn_b200_run_batch; one call in flight per handle. */
typedef struct ncnn_b200_multi ncnn_b200_multi;
int ncnn_b200_multi_load(const char *param_path, const char *bin_path, const ncnn_b200_options *options,
                         const int32_t *devices, int32_t device_count, ncnn_b200_multi **out);
void ncnn_b200_multi_free(ncnn_b200_multi *model);
const char *ncnn_b200_multi_last_error(const ncnn_b200_multi *model);
int32_t ncnn_b200_multi_device_count(const ncnn_b200_multi *model);
int ncnn_b200_multi_run_batch(ncnn_b200_multi *model, int64_t n, const float *const *inputs,
                              float *const *outputs);
/* first[g], count[g] for g < parts: the images of shard g of a batch of n (pure arithmetic, no GPU). */
int ncnn_b200_multi_partition(int64_t n, int32_t parts, int64_t *first, int64_t *count);

/* No counterpart in the reference.  For hosts that are not allowed to allocate on the
 * GPU (a real-time loop after start-up, a sandbox that forbids cudaMalloc, a process whose
 * own pool already owns the whole device): the int8 InnerProduct
 *     y[m][n] = act(float(sum_k Q(x[m][k], input_scale) * weight[n][k]) / (weight_scales[n]*input_scale) + bias[n])
 * on device arrays, with its only scratch (the int8 copy of x) taken from an 8 MiB array
 * built into the library.  It calls no allocation routine.  Limits and rules:
 * m*k <= 8 388 608, otherwise status 5 and a message in ncnn_b200_last_error(NULL); every
 * GPU on which the library's code is loaded (lazily, at the first call on that device: make
 * it at start-up) holds those 8 MiB until exit; calls on one device share the
 * array, so calls that may overlap on the GPU race and must be serialised; the first call
 * on a device resolves the array's address and should happen before any stream capture;
 * the address is cached, so do not call this after cudaDeviceReset() on that device.
 * x is fp32 [m][k], weight int8 [n][k] at any byte alignment, bias fp32 [n] or NULL,
 * y fp32 [m][n]; the arithmetic equals the InnerProduct layer of a loaded int8 model bit
 * for bit. */
int ncnn_b200_inner_product_int8_noalloc(const float *x, const int8_t *weight,
                                         const float *weight_scales, float input_scale,
                                         const float *bias, float *y, int64_t m, int32_t k, int32_t n,
                                         int32_t relu, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* NCNN_B200_H_ */
