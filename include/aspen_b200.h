/*
 * aspen_b200 -- C ABI of the B200 (sm_100a) execution backend for the ASPEN tile-dataflow runtime.
 *
 * Every entry point below replaces the reference function of the same name; a program written
 * against the reference's public header compiles and links against libaspen_b200.so unchanged
 * (include/aspen.h in this tree forwards here).  "ref:" gives the reference declaration and the
 * definition each one stands in for.  Enum VALUES are part of the ABI: they are written as
 * integers into .aspen files (ref: src/apu_file_io.c:451-452) and passed in `order` arrays.
 *
 * All handles are opaque.  Pointer-returning calls give NULL and print to stderr on failure,
 * void calls print and return (ref: include/aspen.h:36, ERROR_PRTF); the last message is also
 * kept for aspen_b200_last_error().  Calls are made from one host thread per dse_group.
 */
#ifndef ASPEN_B200_H_
#define ASPEN_B200_H_

#include <stddef.h>
#include <stdint.h>
#include <sys/types.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ref: include/aspen.h:26-32 -- graph-geometry constants of the reference tiler */
#define MAX_TENSOR_DIMS 8
#define MAX_STRING_LEN 256
#define MAX_PARENT_NINST_NUM (1 << 16)
#define NINST_H_MIN 64
#define NINST_W_MIN 12
#define MEM_ALIGN 32

/* ref: include/aspen.h:50-65 */
typedef enum { NINST_NOT_READY, NINST_READY, NINST_COMPLETED, NUM_NINST_STATES } NINST_STATE;
typedef enum {
    NO_LAYER_TYPE, INPUT_LAYER, CONV_LAYER, FC_LAYER, RESIDUAL_LAYER, BATCHNORM_LAYER, YOLO_LAYER,
    APPEND_LAYER, ACTIVATION_LAYER, MAXPOOL_LAYER, AVGPOOL_LAYER, ROUTE_LAYER, SOFTMAX_LAYER,
    MATMUL_LAYER, LAYERNORM_LAYER, K_ATTENTION_LAYER, V_ATTENTION_LAYER, NUM_LAYER_ELEMENTS
} LAYER_TYPE;
typedef enum {
    OUT_W, OUT_H, OUT_C, BATCH, IN_W, IN_H, IN_C, WEIGHT_W, WEIGHT_H, SUB_C, STRIDE, PADDING,
    DILATION, GROUPS, NUM_HIDDEN, NUM_HEAD, NUM_SEQ, MAT_M, MAT_N, MAT_K, SUB_M, MASKED,
    FORM_BYTES, NUM_PARAM_ELEMENTS
} LAYER_PARAMS;
typedef enum {
    NULL_TENSOR, OUTPUT_TENSOR, INPUT_TENSOR, WEIGHT_TENSOR, BIAS_TENSOR, COL_IDX_TENSOR,
    ANCHOR_TENSOR, BN_VAR_TENSOR, BN_MEAN_TENSOR, BN_WEIGHT_TENSOR, NUM_TENSORS
} LAYER_TENSORS;
typedef enum { PARENT_NONE, PARENT_0, PARENT_1, PARENT_WEIGHT, NUM_PARENT_ELEMENTS } LAYER_PARENTS;
typedef enum {
    NO_ACTIVATION, SIGMOID, LINEAR, TANH, RELU, LEAKY_RELU, ELU, SELU, GELU, GELU_ACCURATE,
    NUM_ACTIVATIONS
} LAYER_ACT;
typedef enum { RPOOL_DNN, RPOOL_LAYER_TYPE, RPOOL_LAYER_IDX, RPOOL_NASM, RPOOL_DSE, NUM_RPOOL_CONDS } RPOOL_CONDS;

/* ref: include/aspen.h:67-73, src/util.c:3-41 */
extern char *ninst_state_str[NUM_NINST_STATES];
extern char *layer_type_str[NUM_LAYER_ELEMENTS];
extern char *param_type_str[NUM_PARAM_ELEMENTS];
extern char *tensor_type_str[NUM_TENSORS];
extern char *parent_type_str[NUM_PARENT_ELEMENTS];
extern char *activation_type_str[NUM_ACTIVATIONS];
extern char *rpool_cond_str[NUM_RPOOL_CONDS];

/* ref: include/aspen.h:75-88 */
typedef struct aspen_dnn_t aspen_dnn_t;
typedef struct aspen_layer_t aspen_layer_t;
typedef struct aspen_tensor_t aspen_tensor_t;
typedef struct ninst_t ninst_t;
typedef struct nasm_t nasm_t;
typedef struct nasm_ldata_t nasm_ldata_t;
typedef struct rpool_t rpool_t;
typedef struct rpool_queue_t rpool_queue_t;
typedef struct rpool_queue_group_t rpool_queue_group_t;
typedef struct dse_t dse_t;
typedef struct dse_group_t dse_group_t;

/* ---- model: cfg + weights -> layer list ------------------------------------------------- */
/* ref: include/aspen.h:90, src/apu.c:6-43.  data_path may be NULL (random +-0.3 weights). */
aspen_dnn_t *apu_create_dnn(char *input_path, char *data_path);
/* ref: include/aspen.h:91, src/apu.c:45-57.  Refused while a nasm still references the dnn. */
void apu_destroy_dnn(aspen_dnn_t *dnn);
/* ref: include/aspen.h:92-93, src/apu_file_io.c:434-809 */
void apu_save_dnn_to_file(aspen_dnn_t *dnn, char *filename);
aspen_dnn_t *apu_load_dnn_from_file(char *filename);

/* ---- tile graph ------------------------------------------------------------------------- */
/* ref: include/aspen.h:95-96, src/apu_nasm.c:601-679.  Tile-count search with the executor in the loop. */
nasm_t *apu_generate_nasm(aspen_dnn_t *dnn, unsigned int batch_size, unsigned int num_iter);
nasm_t *apu_generate_transformer_nasm(aspen_dnn_t *dnn, unsigned int batch_size, unsigned int seq_num, unsigned int num_iter);
/* ref: include/aspen.h:97-98, src/apu_nasm.c:682-751 */
nasm_t *apu_create_nasm(aspen_dnn_t *dnn, unsigned int min_ninst_per_ldata, unsigned int batch_size);
nasm_t *apu_create_transformer_nasm(aspen_dnn_t *dnn, unsigned int min_ninst_per_ldata, unsigned int batch_size, unsigned int seq_num);
/* ref: include/aspen.h:99, src/apu_nasm.c:936-948 */
void apu_destroy_nasm(nasm_t *nasm);
/* ref: include/aspen.h:100-101, src/apu_file_io.c:811-1094 */
nasm_t *apu_load_nasm_from_file(char *filename, aspen_dnn_t *dnn);
void apu_save_nasm_to_file(nasm_t *nasm, char *filename);
/* ref: include/aspen.h:102, src/apu_nasm.c:753-771 */
void apu_reset_nasm(nasm_t *nasm);

/* ---- ready pool ------------------------------------------------------------------------- */
/* ref: include/aspen.h:104-105, src/rpool.c:47-72 */
rpool_t *rpool_init(void);
void rpool_destroy(rpool_t *rpool);
/* ref: include/aspen.h:106, src/rpool.c:167-193 + src/dse.c:443-470.  input_data: packed NHWC
 * ([B][H][W][C]) or [B][S][M] fp32 in HOST memory; it is copied, the caller keeps its buffer. */
void rpool_add_nasm_raw_input(rpool_t *rpool, nasm_t *nasm, void *input_data);
/* ref: include/aspen.h:107, src/rpool.c:195-223.  File holds NCHW fp32; NULL means zeros. */
void rpool_add_nasm(rpool_t *rpool, nasm_t *nasm, char *input_filename);
/* ref: include/aspen.h:108-109, src/rpool.c:262-277 */
void rpool_reset_queue(rpool_t *rpool);
void rpool_reset_nasm(rpool_t *rpool, nasm_t *nasm);

/* ---- scheduling engines ----------------------------------------------------------------- */
/* ref: include/aspen.h:111-113, src/dse.c:110-151.  Here a "dse" is a persistent worker CTA. */
dse_group_t *dse_group_init(unsigned int num_dse);
void dse_group_set_rpool(dse_group_t *dse_group, rpool_t *rpool);
void dse_group_destroy(dse_group_t *dse_group);
/* ref: include/aspen.h:114-116, src/dse.c:234-277.  run is asynchronous, stop is cooperative. */
void dse_group_run(dse_group_t *dse_group);
void dse_group_stop(dse_group_t *dse_group);
void dse_group_run_until_nasm_completion(dse_group_t *dse_group, nasm_t *nasm);
/* ref: include/aspen.h:117-118, src/dse.c:260-289 */
void dse_wait_for_nasm_completion(nasm_t *nasm);
unsigned int dse_check_nasm_completion(nasm_t *nasm);
/* ref: include/aspen.h:119-120, src/dse.c:472-518 + src/apu.c:227-297.  *out_ptr is malloc'd
 * host memory the caller frees; return value is its size in bytes, -1 on bad arguments. */
ssize_t dse_get_ldata_result(nasm_t *nasm, unsigned int ldata_idx, LAYER_PARAMS *order, void **out_ptr);
ssize_t dse_get_nasm_result(nasm_t *nasm, LAYER_PARAMS *order, void **out_ptr);

/* ref: include/aspen.h:122, src/util.c:175-192.  Releases the cached activation arenas. */
void aspen_flush_dynamic_memory(void);

/* ref: include/aspen.h:124-133 */
void print_aspen_build_info(void);
void print_dnn_info(aspen_dnn_t *dnn, int print_data);
void print_layer_info(aspen_layer_t *layer, int print_data);
void print_tensor_info(aspen_tensor_t *tensor, int print_data);
void print_nasm_info(nasm_t *nasm, int print_ninst, int print_data);
void print_ldata_info(nasm_ldata_t *ldata, int print_ninst, int print_data);
void print_ninst_info(ninst_t *ninst, int print_data);
void print_rpool_queue_info(rpool_queue_t *rpool_queue);
void print_rpool_queue_group_info(rpool_queue_group_t *rpool_queue_group);
void print_rpool_info(rpool_t *rpool);

/* ---- additions of this backend (no counterpart in the reference) ------------------------ */

/* Last error text of the calling process ("" if none). */
const char *aspen_b200_last_error(void);

/* Engine status of the most recent run of a dse group: 0 ok, otherwise an ASPEN_B200_ERR_* code
 * written by the device scheduler when a bounded wait ran out (the kernel then returns instead
 * of spinning). */
#define ASPEN_B200_OK 0
#define ASPEN_B200_ERR_STALL 1      /* ready-queue wait ran out: graph cannot make progress   */
#define ASPEN_B200_ERR_PIPE 2       /* an in-kernel pipeline barrier wait ran out             */
#define ASPEN_B200_ERR_CUDA 3       /* a CUDA runtime call failed (see aspen_b200_last_error)  */
int aspen_b200_group_status(dse_group_t *dse_group);

/* Tiler profile.  The reference's constants (64-row / 12-column quanta, 1e8 flop per tile) shape
 * tiles for an 8x12 AVX2 register block; profile 1 uses 128-row / 128-column quanta so a tile is
 * whole 128 x 128 tensor-core blocks.  Tile VALUES do not depend on the profile.  Affects nasms
 * created afterwards.  0 = reference geometry (default), 1 = B200 geometry. */
void aspen_b200_set_tile_profile(int profile);
void aspen_b200_set_tile_quanta(unsigned int h_min, unsigned int w_min, unsigned int flop_per_ninst);

/* Tile-shape search for the GPU at hand (the B200 counterpart of apu_generate_nasm, ref src/apu_nasm.c:578-679,
 * which tunes the tile count for the CPU kernels): tries tensor-core shaped quanta (128 x 128, 256 x 128,
 * 128 x 256) times 100 ... 296 tiles per layer, times each candidate on the device, and returns a nasm built
 * with the fastest.  seq_num = 0 for image networks.  chosen (may be NULL) receives {row quantum, column
 * quantum, min_ninst_per_ldata}.  The global tile profile is left as it was.  Needs an sm_100 GPU. */
nasm_t *aspen_b200_generate_nasm(aspen_dnn_t *dnn, unsigned int batch_size, unsigned int seq_num, unsigned int *chosen);

/* Arithmetic of the contraction tiles for dse groups created afterwards:
 * 0 = TF32 operands on tcgen05 tensor cores, fp32 accumulate (default);
 * 1 = fp32 FFMA validation mode. */
void aspen_b200_set_precision(int mode);

/* CUDA device used by objects created afterwards on the calling thread (default: current). */
int aspen_b200_set_device(int device);

/* Read-only views used by the parity tests and the benchmark. */
unsigned int aspen_b200_dnn_num_layers(aspen_dnn_t *dnn);
void aspen_b200_dnn_layer_params(aspen_dnn_t *dnn, unsigned int layer_idx, unsigned int *params_out /*[NUM_PARAM_ELEMENTS]*/);
int aspen_b200_dnn_layer_type(aspen_dnn_t *dnn, unsigned int layer_idx);
unsigned int aspen_b200_nasm_num_ldata(nasm_t *nasm);
unsigned int aspen_b200_nasm_num_ninst(nasm_t *nasm);
uint64_t aspen_b200_nasm_total_flops(nasm_t *nasm);
/* out[12]: type, activation, H, W, stride, tile H, tile W, num_ninst, flop_per_output, parent0, parent1, mem bytes */
void aspen_b200_nasm_ldata_info(nasm_t *nasm, unsigned int ldata_idx, unsigned int *out);
/* out[7]: pos H, pos W, tile H, tile W, num parents, num children, num_input_pos */
void aspen_b200_nasm_ninst_info(nasm_t *nasm, unsigned int ninst_idx, unsigned int *out);
/* Copies up to `cap` parent (children) ninst indices; returns the full count. */
unsigned int aspen_b200_nasm_ninst_parents(nasm_t *nasm, unsigned int ninst_idx, unsigned int *out, unsigned int cap);
unsigned int aspen_b200_nasm_ninst_children(nasm_t *nasm, unsigned int ninst_idx, unsigned int *out, unsigned int cap);
/* Packed column-major copy (H contiguous x W columns) of one layer's activations after a run;
 * returns element count or -1. */
long aspen_b200_nasm_get_ldata_packed(nasm_t *nasm, unsigned int ldata_idx, float *out);

/* Timed execution for benchmarks: runs the group's rpool `iters` times (re-arming every nasm in
 * it between runs, as rpool_reset_nasm does) and returns the device time of the runs in
 * milliseconds measured with CUDA events on the group's stream; *launches_out (may be NULL) gets
 * the number of kernel launches issued.  Returns a negative value on error. */
double aspen_b200_group_time_runs(dse_group_t *dse_group, unsigned int warmup, unsigned int iters, unsigned long long *launches_out);

/* Service mode of a dse group.  The reference's DSE threads live from dse_group_run to dse_group_stop and serve
 * whatever rpool_add_nasm brings in the meantime (ref src/dse.c:20-108, 215-232; src/rpool.c:390-685).  With the mode
 * on, this library does the same on the device: dse_group_run launches ONE scheduler kernel over the graphs of the
 * pool and that kernel stays resident; rpool_add_nasm / rpool_add_nasm_raw_input / aspen_b200_rpool_add_nasm_tokens /
 * rpool_reset_nasm on a graph it serves upload the input and ask for one more pass of the graph (a graph takes one
 * request at a time: a second request first waits for the pass that is owed); dse_wait_for_nasm_completion waits for
 * the pass last asked for; dse_get_nasm_result and the layer readers copy with the copy engine; dse_group_stop ends
 * the kernel once nothing is running or owed.  Passes of different graphs overlap on the SMs, so the late, narrow
 * layers of one request run next to the early, wide layers of the next.  The input layer's tiles run on the device
 * (scatter, TF32 rounding, embedding gather), so nothing but copies is issued while the kernel is resident; calls
 * that must allocate or free device memory (a graph's first use, its destruction) stop the kernel first and the next
 * run or wait starts it again.  Left idle for 20 ms (ASPEN_B200_IDLE_MS) the kernel leaves by itself.
 * Off by default: each dse_group_run then launches the scheduler for the graphs armed at that moment.
 * Returns 0, or -1 on error.  Graphs that use the fused attention tile are not served in this mode. */
int aspen_b200_dse_group_set_service(dse_group_t *dse_group, int on);

/* Timed execution in service mode: `passes` passes dealt round robin to the graphs of the group's rpool (inputs as
 * they are on the device), inside service launches that end when the passes are complete; returns the device time in
 * milliseconds between CUDA events on the group's stream, a negative value on error. */
double aspen_b200_group_time_passes(dse_group_t *dse_group, unsigned int warmup, unsigned int passes, unsigned long long *launches_out);

/* Time accounting of the device scheduler (replaces the reference's wall-clock probes,
 * ref src/util.c:490-539).  Active when the environment variable ASPEN_B200_PROFILE is set before
 * dse_group_init.  out[516], summed over all worker CTAs since the last call: [0] scheduler polls
 * made with nothing in flight, [1] ns spent on completion and child updates, [2 + l] ns the executor
 * warps spent on tiles of layer l (l modulo 256), [258 + l] number of tiles of layer l, [515] ns the
 * executor warps waited for a tile.  Returns 0, or -1 when inactive. */
int aspen_b200_group_profile(dse_group_t *dse_group, unsigned long long *out, unsigned int *n_ctas);

/* No counterpart in the reference: its transformer cfgs start at the hidden states ([net] M=768; ref
 * files/bert_base/bert_base_aspen.cfg, files/gpt2_124M/gpt2_124M_aspen.cfg) and leave the embedding lookup to the
 * caller.  aspen_b200_dnn_set_embedding registers the tables of a dnn (host pointers, copied): token_table
 * [vocab][M] and position_table [max_pos][M] or NULL, M = the width of the dnn's first layer; call it before the
 * dnn's first graph is uploaded.  aspen_b200_rpool_add_nasm_tokens then stands in for rpool_add_nasm_raw_input:
 * token_ids is a host array [batch][seq] of int32; column b * seq + s of layer 0 becomes
 * token_table[id] + position_table[s], gathered on the device.  The rpool must already belong to a dse group.
 * A tied output head needs nothing new: it is a [matmul] layer whose weights are the token table (M = vocab). */
int aspen_b200_dnn_set_embedding(aspen_dnn_t *dnn, const float *token_table, unsigned int vocab, const float *position_table,
                                 unsigned int max_pos);
void aspen_b200_rpool_add_nasm_tokens(rpool_t *rpool, nasm_t *nasm, const int *token_ids);

/* No counterpart in the reference, whose DSEs free a layer's buffer once its child layers are complete
 * (ref src/dse.c:84-92), so that only the last layer can be read after a run.  This library keeps every layer
 * readable by default (dse_get_ldata_result on any layer).  keep = 0 gives that up for the layers whose output
 * only feeds a residual add fused into their own epilogue (the expand convolutions of ResNet bottlenecks, the
 * attention / FFN output projections of a transformer): their pre-add values are then never written to memory;
 * reading such a layer afterwards returns zeros or stale data.  Every other layer, and the result, are unchanged
 * bit for bit.  Applies to graphs whose device image is built after the call (first rpool_add_nasm on a group);
 * the environment variable ASPEN_B200_HIDDEN_STATES=0 selects the same for programs that cannot call this. */
void aspen_b200_set_hidden_states(int keep);

/* No counterpart in the reference.  One matmul layer, out[n][m] = act(bias[m] + sum_k w[m][k] * x[n][k])
 * in fp32 FMA arithmetic, run as 128 x 128 tiles by the same persistent scheduler kernel as every
 * other call -- but WITHOUT ALLOCATING ANYTHING.  It is for callers that are not allowed to call
 * cudaMalloc: plug-ins of a serving runtime that fixes all memory pools at start-up and treats a later
 * allocation as a bug, and loops that cannot afford the device-wide synchronisation an allocation
 * implies.  All pointers are DEVICE pointers the caller owns: x [n_cols][k], w [m][k],
 * bias [m] or NULL, out [n_cols][m], rows contiguous; cuda_stream is a cudaStream_t (NULL = default).
 * Everything else the scheduler needs (tile descriptors, ready queue, counters, status) lives in one
 * fixed array in device memory that every GPU holds from the moment the library is loaded until exit
 * (about 180 KB).  Hence:
 *   - at most ASPEN_B200_NOALLOC_MAX_TILES tiles, i.e. ceil(m/128) * ceil(n_cols/128) <= 4096; a larger
 *     call fails with -2 and changes nothing;
 *   - all calls on one GPU share the array, which still holds the previous call's data: each call
 *     rewrites what it reads (counters and queue start from zero), and calls that overlap on the GPU
 *     -- two streams, two host threads -- corrupt each other.  Serialise them;
 *   - the first call on a device resolves the array's device address; make that call before any
 *     stream capture begins.
 * The call waits for its own work on `cuda_stream` (it synchronises that stream to read the scheduler's
 * status back) and returns after the work has finished.  Returns 0, -1 bad arguments, -2 too large, -3 CUDA
 * error, -4 the scheduler reported an error (see aspen_b200_last_error). */
#define ASPEN_B200_NOALLOC_MAX_TILES 4096
int aspen_b200_matmul_noalloc(const float *x_dev, const float *w_dev, const float *bias_dev, float *out_dev,
                              unsigned int n_cols, unsigned int k, unsigned int m, int activation, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* ASPEN_B200_H_ */
