/*
 * TEST INFRASTRUCTURE ONLY -- never linked into or called from the product library.
 *
 * Driver around the UNMODIFIED ASPEN reference sources.  It is compiled together with the
 * reference's own src/*.c (see oracle/Makefile) into oracle/_ref/libaspen_ref.so and gives the
 * parity tests three things the reference's public API does not:
 *
 *   1. refwalk_run():   a layer-by-layer walk that calls the reference's own tiled_* kernels
 *                       (src/tiled_kernels.c) once per ninst and keeps every layer's out_mat alive,
 *                       so hidden states can be compared (the threaded DSE path frees intermediate
 *                       buffers, src/dse.c:84-92).
 *   2. refwalk_*_info(): read-only accessors for the tile geometry the reference's tiler
 *                       (src/apu_nasm.c:1025-1182) produced, so the product's tiler can be diffed.
 *   3. refbench_dse():  the timing loop of the reference's CLI driver (main.c:116-123) around the
 *                       reference's pthread DSE workers -- the timed CPU baseline.
 *
 * Nothing here restates reference code; it only calls it.
 */
#include "aspen.h"
#include "apu.h"
#include "nasm.h"
#include "dse.h"
#include "rpool.h"
#include "kernels.h"
#include <omp.h>

void ninst_find_input_pos_idx (ninst_t *ninst);

#define WALK_SCRATCH_BYTES (32u * 1024u * 1024u)

static void run_one_ninst (ninst_t *ninst, dse_t *dse)
{
    /* same dispatch as dse_schedule, src/dse.c:39-79 */
    switch (ninst->ldata->layer->type)
    {
        case CONV_LAYER: tiled_conv2d (ninst, dse); break;
        case MAXPOOL_LAYER: tiled_maxpool2d (ninst, dse); break;
        case AVGPOOL_LAYER: tiled_avgpool2d (ninst, dse); break;
        case FC_LAYER: tiled_fully_connected (ninst, dse); break;
        case RESIDUAL_LAYER: tiled_residual (ninst, dse); break;
        case SOFTMAX_LAYER: tiled_softmax (ninst, dse); break;
        case YOLO_LAYER: tiled_yolo (ninst, dse); break;
        case APPEND_LAYER: tiled_append (ninst, dse); break;
        case MATMUL_LAYER: tiled_matmul (ninst, dse); break;
        case LAYERNORM_LAYER: tiled_layernorm (ninst, dse); break;
        case K_ATTENTION_LAYER: tiled_k_attention (ninst, dse); break;
        case V_ATTENTION_LAYER: tiled_v_attention (ninst, dse); break;
        default: break;
    }
}

/* Build the tile list only (no parent search: minutes at batch 32).  The walk needs
 * num_input_pos, which the parent search would have set (src/apu_nasm.c:37-46). */
nasm_t *refwalk_create_nasm (aspen_dnn_t *dnn, unsigned int min_ninst, unsigned int batch, unsigned int seq)
{
    nasm_t *nasm = apu_create_nasm_without_finding_ninst_parents (dnn, APU_GENERATION_NUM_FLOPS, batch, min_ninst, seq);
    for (unsigned int i = 0; i < nasm->num_ninst; i++)
        ninst_find_input_pos_idx (&nasm->ninst_arr[i]);
    return nasm;
}

/* input: packed NHWC (or [B][S][M]) fp32, as rpool_add_nasm_raw_input takes it. */
int refwalk_run (nasm_t *nasm, void *input, int num_threads)
{
    if (nasm == NULL || input == NULL)
        return -1;
    if (num_threads < 1)
        num_threads = 1;
    for (unsigned int i = 0; i < nasm->num_ldata; i++)
        alloc_ldata_out_mat (&nasm->ldata_arr[i]);
    copy_buffer_to_ldata_out_mat (&nasm->ldata_arr[0], input);
    dse_t *dses = calloc (num_threads, sizeof (dse_t));
    for (int t = 0; t < num_threads; t++)
        dses[t].scratchpad = aspen_calloc (WALK_SCRATCH_BYTES, 1);
    for (unsigned int i = 1; i < nasm->num_ldata; i++)
    {
        nasm_ldata_t *ldata = &nasm->ldata_arr[i];
        #pragma omp parallel for num_threads(num_threads) schedule(dynamic, 1)
        for (unsigned int j = 0; j < ldata->num_ninst; j++)
            run_one_ninst (&ldata->ninst_arr_start[j], &dses[omp_get_thread_num ()]);
    }
    for (int t = 0; t < num_threads; t++)
        aspen_free (dses[t].scratchpad);
    free (dses);
    return 0;
}

/* Packed column-wise copy (H contiguous, W columns) of one layer's activations. */
long refwalk_get_ldata (nasm_t *nasm, unsigned int idx, float *out)
{
    if (nasm == NULL || idx >= nasm->num_ldata || nasm->ldata_arr[idx].out_mat == NULL)
        return -1;
    nasm_ldata_t *ldata = &nasm->ldata_arr[idx];
    copy_ldata_out_mat_to_buffer (ldata, out);
    return (long) ldata->out_mat_dims[OUT_H] * ldata->out_mat_dims[OUT_W];
}

unsigned int refwalk_num_ldata (nasm_t *nasm) { return nasm->num_ldata; }
unsigned int refwalk_num_ninst (nasm_t *nasm) { return nasm->num_ninst; }
unsigned long refwalk_total_flops (nasm_t *nasm) { return nasm->total_flops; }

/* out[0..11]: layer type, activation, out_mat H, W, stride, tile H, tile W, num_ninst,
 * flop_per_output, parent0 idx, parent1 idx, out_mat_mem_size (bytes, truncated to 32 bit). */
void refwalk_ldata_info (nasm_t *nasm, unsigned int idx, unsigned int *out)
{
    nasm_ldata_t *l = &nasm->ldata_arr[idx];
    out[0] = l->layer->type;
    out[1] = l->layer->activation;
    out[2] = l->out_mat_dims[OUT_H];
    out[3] = l->out_mat_dims[OUT_W];
    out[4] = l->out_mat_stride;
    out[5] = l->ninst_tile_dims[OUT_H];
    out[6] = l->ninst_tile_dims[OUT_W];
    out[7] = l->num_ninst;
    out[8] = l->flop_per_output;
    out[9] = l->parent_ldata_idx_arr[PARENT_0];
    out[10] = l->parent_ldata_idx_arr[PARENT_1];
    out[11] = (unsigned int) l->out_mat_mem_size;
}

/* out[0..6]: pos H, pos W, tile H, tile W, num parents, num children, num_input_pos */
void refwalk_ninst_info (nasm_t *nasm, unsigned int idx, unsigned int *out)
{
    ninst_t *n = &nasm->ninst_arr[idx];
    out[0] = n->out_mat_pos[OUT_H];
    out[1] = n->out_mat_pos[OUT_W];
    out[2] = n->tile_dims[OUT_H];
    out[3] = n->tile_dims[OUT_W];
    out[4] = n->num_parent_ninsts;
    out[5] = n->num_child_ninsts;
    out[6] = n->num_input_pos;
}

void refwalk_layer_params (aspen_dnn_t *dnn, unsigned int idx, unsigned int *out)
{
    for (int i = 0; i < NUM_PARAM_ELEMENTS; i++)
        out[i] = dnn->layers[idx].params[i];
}
unsigned int refwalk_num_layers (aspen_dnn_t *dnn) { return dnn->num_layers; }

/* Reference timing loop, main.c:116-123.  Returns seconds per iteration (wall). */
double refbench_dse (nasm_t *nasm, void *input, unsigned int num_dse, unsigned int warmup, unsigned int iters)
{
    rpool_t *rpool = rpool_init ();
    dse_group_t *dse_group = dse_group_init (num_dse);
    dse_group_set_rpool (dse_group, rpool);
    rpool_add_nasm_raw_input (rpool, nasm, input);
    struct timeval t0, t1;
    double total = 0;
    for (unsigned int i = 0; i < warmup + iters; i++)
    {
        if (i == warmup)
            gettimeofday (&t0, NULL);
        if (i != 0)
        {
            rpool_reset_queue (rpool);
            rpool_reset_nasm (rpool, nasm);
        }
        dse_group_run (dse_group);
        dse_wait_for_nasm_completion (nasm);
        dse_group_stop (dse_group);
    }
    gettimeofday (&t1, NULL);
    total = (t1.tv_sec - t0.tv_sec) + (t1.tv_usec - t0.tv_usec) * 1e-6;
    dse_group_destroy (dse_group);
    rpool_destroy (rpool);
    return total / (iters > 0 ? iters : 1);
}
