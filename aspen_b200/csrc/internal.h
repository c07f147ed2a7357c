// Internal data model of libaspen_b200: what the opaque handles of include/aspen_b200.h point to.
#pragma once
#include "../../include/aspen_b200.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

struct DeviceNasm;   // engine.cu
struct DeviceDnn;    // engine.cu
struct Engine;       // engine.cu

// A host tensor: dims are looked up by LAYER_PARAMS id, data is packed in data_dim_order.
struct aspen_tensor_t {
    unsigned int num_dims = 0;
    LAYER_PARAMS data_dim_order[MAX_TENSOR_DIMS] = {};
    unsigned int dims[NUM_PARAM_ELEMENTS] = {};
    unsigned int num_elements = 0;
    unsigned int element_size = 4;
    void *data = nullptr;
};

struct aspen_layer_t {
    aspen_dnn_t *dnn = nullptr;
    unsigned int layer_idx = 0;
    LAYER_TYPE type = NO_LAYER_TYPE;
    LAYER_ACT activation = NO_ACTIVATION;
    aspen_layer_t *parent_layers[NUM_PARENT_ELEMENTS] = {};
    unsigned int params[NUM_PARAM_ELEMENTS] = {};
    aspen_tensor_t *tensors[NUM_TENSORS] = {};
};

// Weights are kept on the host in the canonical contraction layout the device consumes:
// WEIGHT_TENSOR is [rows = OUT_C or MAT_M][K], K ordered (kh, kw, ic) for conv, (ih, iw, ic) for
// connected layers and plain k for matmul.  (The reference re-packs to [M/8][K][8] for its AVX2
// micro-kernel, src/apu.c:14-40; that layout only exists here inside the .aspen file codec.)
struct aspen_dnn_t {
    char name[MAX_STRING_LEN] = {};
    unsigned int element_size = 4;
    std::vector<aspen_layer_t> layers;
    unsigned int num_layers = 0;
    std::atomic<unsigned int> ref_nasms{0};
    DeviceDnn *dev[16] = {};   // per-CUDA-device weight copies, created on first use
    // Embedding tables of a transformer whose cfg starts at the hidden states (aspen_b200_dnn_set_embedding):
    // token_table [vocab][M], position_table [max_pos][M] (may be empty).
    std::vector<float> emb_token, emb_position;
    unsigned int emb_vocab = 0, emb_max_pos = 0, emb_width = 0;
};

struct ninst_t {
    nasm_ldata_t *ldata = nullptr;
    NINST_STATE state = NINST_NOT_READY;
    unsigned int ninst_idx = 0;
    unsigned int out_mat_pos[2] = {};   // indexed by OUT_W (0) / OUT_H (1)
    unsigned int tile_dims[2] = {};
    std::vector<unsigned int> parent_ninst_idx;
    std::vector<unsigned int> child_ninst_idx;
    std::vector<unsigned int> extra_parent_idx;   // true dependencies missing from the reference's list (device only)
    unsigned int num_input_pos = 0;
};

struct nasm_ldata_t {
    nasm_t *nasm = nullptr;
    aspen_layer_t *layer = nullptr;
    unsigned int parent_ldata_idx_arr[NUM_PARENT_ELEMENTS] = {};
    std::vector<unsigned int> child_ldata_idx;
    unsigned int num_child_ldata = 0;
    unsigned int flop_per_output = 1;
    unsigned int out_mat_dims[2] = {};
    unsigned int out_mat_stride = 0;
    size_t out_mat_mem_size = 0;
    unsigned int ninst_tile_dims[2] = {};
    unsigned int ninst_start = 0;
    unsigned int num_ninst = 0;
};

struct TileQuanta {
    unsigned int h_min = NINST_H_MIN;
    unsigned int w_min = NINST_W_MIN;
    unsigned int flop_per_ninst = 100000000u;
};

struct nasm_t {
    unsigned int nasm_id = 0;
    aspen_dnn_t *dnn = nullptr;
    unsigned int batch_size = 1;
    unsigned int tr_seq_len = 0;
    std::vector<nasm_ldata_t> ldata;
    std::vector<ninst_t> ninst;
    unsigned int num_ldata = 0;
    unsigned int num_ninst = 0;
    unsigned int min_ninst_per_ldata = 0;
    unsigned int flop_per_ninst = 0;
    size_t total_flops = 0;
    uint64_t true_flops = 0;
    TileQuanta quanta;
    bool has_graph = false;
    // runtime side
    std::atomic<unsigned int> completed{0};
    DeviceNasm *dev = nullptr;     // device image (arena, descriptors, counters)
    rpool_t *rpool = nullptr;      // pool this nasm was added to
    std::vector<float> staged_input;   // input given before the pool had a dse group
    bool staged = false;
};

struct rpool_t {
    std::vector<nasm_t *> nasms;
    std::atomic<unsigned int> ref_dses{0};
    Engine *engine = nullptr;      // set by the dse group that serves this pool
};

struct dse_group_t {
    unsigned int num_dses = 0;
    rpool_t *rpool = nullptr;
    Engine *engine = nullptr;
    int precision = 0;
    int device = 0;
};

// ---- helpers ---------------------------------------------------------------------------
void aspen_error(const char *file, int line, const char *fmt, ...);
#define ASPEN_ERR(...) aspen_error(__FILE__, __LINE__, __VA_ARGS__)

static inline size_t round_up(size_t num, size_t div) { return (num / div + (num % div != 0)) * div; }

// cfg.cpp
aspen_dnn_t *parse_cfg_file(const char *path);
// dnn.cpp
aspen_tensor_t *tensor_create(const unsigned int *params, const LAYER_PARAMS *order, int num_dims, unsigned int elem);
void tensor_destroy(aspen_tensor_t *t);
unsigned int tensor_idx_from_pos(const aspen_tensor_t *t, const unsigned int *pos);
void tensor_pos_from_idx(const aspen_tensor_t *t, unsigned int idx, unsigned int *pos);
unsigned int layer_contraction_k(const aspen_layer_t *l);
unsigned int layer_weight_rows(const aspen_layer_t *l);
// tiler.cpp
extern TileQuanta g_quanta;

// Output pixels per block of a convolution staged by strided TMA boxes, chosen so that a block is whole output
// rows of one sample (or whole samples when a sample has at most 128 pixels): the block is then a single box.
inline unsigned conv_block_width(unsigned OW, unsigned OH) {
    if (OW == 0 || OH == 0 || OW > 128) return 128;
    if (OW * OH <= 128) return (128 / (OW * OH)) * OW * OH;
    unsigned k = 1;
    for (unsigned d = 1; d <= OH && d * OW <= 128; d++)
        if (OH % d == 0) k = d;
    return k * OW;
}
// The convolutions that get that staging when tiles are whole MMA blocks (column quantum 128): IC a multiple of
// 32 and neither a 1x1 stride-1 layer (plain 2-D boxes) nor a stride-1 "same" layer (shifted box + fix-up).
inline bool conv_uses_row_blocks(const aspen_layer_t *l) {
    if (l->type != CONV_LAYER) return false;
    const unsigned *p = l->params;
    const unsigned s = p[STRIDE] ? p[STRIDE] : 1;
    if (p[IN_C] % 32 != 0 || p[OUT_W] > 128 || p[OUT_W] * s > 256 || s > 8) return false;
    if (p[WEIGHT_H] == 1 && p[WEIGHT_W] == 1 && s == 1 && p[PADDING] == 0) return false;
    if (s == 1 && p[OUT_H] == p[IN_H] && p[OUT_W] == p[IN_W] && p[WEIGHT_H] == p[WEIGHT_W] && 2 * p[PADDING] + 1 == p[WEIGHT_H]) return false;
    return true;
}
void tiler_init_ldata(nasm_t *nasm, nasm_ldata_t *ld, aspen_layer_t *layer);
void tiler_init_ninst(nasm_ldata_t *ld, ninst_t *ni, unsigned int ninst_idx);
void out_mat_pos_from_tensor_pos(const nasm_ldata_t *ld, const unsigned int *tpos, unsigned int *mpos);
void tensor_pos_from_out_mat_pos(const nasm_ldata_t *ld, const unsigned int *mpos, unsigned int *tpos);
nasm_t *nasm_create_tiles(aspen_dnn_t *dnn, unsigned int flop_per_ninst, unsigned int batch, unsigned int min_ninst, unsigned int seq);
// graph.cpp
void graph_find_parents(nasm_t *nasm);
void graph_set_children(nasm_t *nasm);
// engine.cu (the only translation unit that touches CUDA)
int engine_current_device();
Engine *engine_create(int device, int precision, unsigned int num_dse_hint);
void engine_destroy(Engine *e);
int engine_attach_nasm(Engine *e, nasm_t *nasm, const void *input_host);   // upload image + input
void engine_detach_nasm(nasm_t *nasm);
int engine_set_input(nasm_t *nasm, const void *input_host);
int engine_set_tokens(nasm_t *nasm, const int *token_ids_host);   // layer 0 = embedding rows of the ids, gathered on the device
int engine_rearm(Engine *e, nasm_t *nasm);
int engine_set_service(Engine *e, int on);                       // service mode: one resident kernel serves pass after pass
bool engine_in_service(Engine *e);
int engine_service_tokens(Engine *e, nasm_t *nasm, const int *token_ids_host);
double engine_time_passes(Engine *e, const std::vector<nasm_t *> &nasms, unsigned int warmup, unsigned int passes, unsigned long long *launches);
int engine_run(Engine *e, const std::vector<nasm_t *> &nasms);
int engine_stop(Engine *e);
int engine_wait_nasm(nasm_t *nasm);
unsigned int engine_poll_nasm(nasm_t *nasm);
int engine_status(Engine *e);
long engine_read_ldata(nasm_t *nasm, unsigned int ldata_idx, float *out_packed);
double engine_time_runs(Engine *e, const std::vector<nasm_t *> &nasms, unsigned int warmup, unsigned int iters, unsigned long long *launches);
void engine_release_dnn(aspen_dnn_t *dnn);
void engine_flush();
int engine_read_profile(Engine *e, unsigned long long *out, unsigned *n_ctas);
