// Flattened device image of a tile graph (nasm) and the scheduler's control block.
// Shared by the host uploader (engine.cu) and the kernels.
#pragma once
#include <cstdint>

// Layer types / activations use the ABI enum values of include/aspen_b200.h.

struct LayerDev {
    int type;                 // LAYER_TYPE
    int act;                  // LAYER_ACT
    float *out;               // own activation matrix: column-major, H rows contiguous, W columns
    unsigned ldc, H, W;       // column stride (floats), logical rows, columns
    const float *in0;         // PARENT_0 activations
    unsigned ld0, H0;
    const float *in1;         // PARENT_1 activations
    unsigned ld1, H1;
    const float *weight;      // [rows][Kpad] fp32, K contiguous, zero padded; layernorm: gain[rows]
    const float *bias;        // [rows]
    unsigned K, Kpad, rows;
    unsigned IC, IH, IW, OH, OW, KH, KW, stride, pad;     // conv / pool geometry
    unsigned seq, heads, hd, masked;                     // attention
    unsigned p_out_c, p_in_c, p_stride;                  // yolo / append raw cfg parameters
    const float *anchors;
    int wmap;                 // tensor map of the W-side operand (weights, or PARENT_1 for attention keys), -1 if none
    int amap;                 // tensor map of the X-side operand (PARENT_0 activations), -1 if gathered
    unsigned a_kind, b_kind;  // operand staging, see tiles_tc.cuh
    unsigned a_vec4;          // activation rows can be fetched in 16-byte pieces (IC % 4 == 0 ...)
    unsigned round_out;       // store outputs rounded to TF32 (nearest): a tensor-core layer reads them
    unsigned PH;              // A_TMA_ROWS: rows per sample of the zero-padded copy of the input image
    unsigned bw;              // tile columns per accumulator block: 128, or whole output rows / samples (A_TMA_IM2COL, one box)
    unsigned one_box;         // A_TMA_IM2COL: index of the single tensor map that covers a block (bw != 128)
    // A residual layer fused into this (convolution / matmul) layer's epilogue: besides its own output the tile
    // also writes res_out = act(own + res_in) for the same region.  res_out == nullptr: nothing fused.
    const float *res_in;
    float *res_out;
    unsigned res_ld_in, res_ld_out;
    int res_act;
    unsigned res_round;
    unsigned res_elide;       // the layer's own (pre-add) output has no other reader and is not written
    int resmap;               // tensor map of res_in (32 x 32 boxes) when the epilogue fetches it by TMA, else -1
    // A layer whose output is the value operand of an attention_v layer also writes it transposed ([feature][token],
    // tokens contiguous): that copy is what the attention tile's TMA reads as a K-major operand.  nullptr: no copy.
    float *vt_out;
    unsigned vt_ld;
    // attention_v layer that computes its own probabilities (attention_k fused into it, see tc::tile_attention):
    // tensor maps of the query and key projections; where the attention_k layer's matrix is still to be written, its
    // address, column stride and rounding flag.
    unsigned att_fused;
    int att_qmap, att_kmap;
    float *att_p_out;
    unsigned att_p_ld, att_p_round;
};

struct TileDev {
    unsigned layer;
    unsigned pos_h, pos_w;    // position in the layer's output matrix
    unsigned tile_h, tile_w;  // clipped extents
    unsigned child_off, child_cnt;
    unsigned need;            // number of parent tiles (true dependencies)
    unsigned flags;           // TILE_WRITTEN_BY_PARENTS
};

// The tile's values were already written by the tiles it depends on (a residual layer fused into its
// producer): the scheduler completes it as soon as it is ready, no executor runs it.
#define TILE_WRITTEN_BY_PARENTS 1u

// Service mode: the layer-0 tiles run on the device and turn what the host uploaded into the layer's activation
// matrix, so a graph's next pass can start inside the running kernel.
struct InputDev {
    const float *stage;       // packed [column][rows] copy as uploaded; nullptr when the upload goes straight into layer 0
    const int *ids;           // token ids as uploaded (one per column), nullptr otherwise
    const float *emb_tok, *emb_pos;
    unsigned emb_vocab, emb_seq;
    float *padded;            // zero-padded [sample][PH][PW][4] copy of the image (A_TMA_ROWS), nullptr otherwise
    unsigned IC, IH, IW, PH, PW, pad;
    unsigned round;           // values are rounded to TF32 (nearest)
};

// words of NasmDev::svc
#define SVC_TARGET 0u         // written by the host: number of the last pass asked for
#define SVC_STARTED 1u        // number of the last pass started
#define SVC_IDLE 2u           // 1: no pass in progress
#define SVC_COUNT 3u          // tiles completed since the kernel was launched

struct NasmDev {
    const LayerDev *layers;
    const TileDev *tiles;
    const unsigned *children;        // CSR payload: (local child tile id, count that child waits for) pairs
    unsigned *dep;                   // [n_tiles] parents completed so far
    const unsigned *dep_init;        // [n_tiles] parents that are input tiles (complete when armed)
    unsigned *layer_done;            // [n_layers] tiles completed per layer
    const unsigned *layer_tiles;     // [n_layers]
    const unsigned *init_ready;      // local ids of tiles runnable right after arming
    unsigned *layers_completed;      // single counter
    const unsigned *layer_done_init; // [n_layers] tiles that count as complete when armed (layer 0: all; bypassed tiles)
    unsigned layers_done_init;       // layers complete when armed
    volatile unsigned *completed;    // mapped host flag, set when every layer is complete
    const void *wmaps;               // CUtensorMap[]
    unsigned n_tiles, n_layers, n_init, n_input_tiles;   // n_input_tiles: every tile complete when armed (input + bypassed)
    unsigned tile_base;              // global id of local tile 0 in this run
    unsigned queue_base;             // where this graph's initial ready tiles go in the queue
    // service mode
    unsigned *svc;                   // SVC_* words in device memory
    unsigned svc_base;               // passes complete when the kernel was launched
    unsigned n_exec;                 // tiles that complete in one pass (every tile but the bypassed ones)
    unsigned n_input;                // layer-0 tiles (local ids 0 .. n_input-1): the seeds of a pass
    InputDev input;
};

struct CtrlDev {
    unsigned head;           // next ticket to hand out
    unsigned tail;           // next free queue slot
    unsigned done;           // tiles completed (input tiles included)
    unsigned total;          // tiles in this run
    unsigned cap;            // queue capacity (== total)
    unsigned abort;          // set with a status code: everybody leaves
    unsigned stop;           // host request: leave after the current tile
    unsigned n_nasm;
    unsigned long long stall_ns;   // no-progress window after which a wait gives up
    unsigned long long pipe_ns;    // time budget of in-kernel pipeline waits
    // service mode
    unsigned svc_stop;       // host request: leave once no pass is running or asked for
    unsigned svc_close;      // set by the device: everybody leaves (no error)
    unsigned busy;           // graphs with a pass in progress
    unsigned svc_ahead;      // a busy CTA lines up a second tile when at least this many ready tiles wait unclaimed (0: never)
    unsigned long long idle_ns;    // leave after this long without a pass in progress
};

struct StatusHost {          // mapped host memory
    volatile unsigned status;        // ASPEN_B200_ERR_*
    volatile unsigned info0, info1;  // where it gave up (tile id / barrier id)
    volatile unsigned tiles_done;
};

#define ASPEN_TILE_NONE 0xffffffffu
