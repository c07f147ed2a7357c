/* A C program written the way the reference's callers are (its main.c and examples/ programs):
 * it includes "aspen.h" and nothing else, and leans on what that header brings along -- FILE,
 * struct timeval / gettimeofday, strcmp, atoi, the PRTF macros.  The tests compile and link it
 * against libaspen_b200.so (no GPU needed for that) and, on a GPU, run it and compare the file it
 * writes with the same network driven through the Python binding.
 *
 *   drop_in_caller <cfg> <weights.bin> <input NCHW fp32 file | -> <batch> <iterations> <nasm file> <output file>
 */
#include "aspen.h"

static double now_sec(void)
{
    struct timeval tv;
    gettimeofday(&tv, NULL);
    return (double)tv.tv_sec + (double)tv.tv_usec * 1e-6;
}

int main(int argc, char **argv)
{
    if (argc != 8) {
        PRTF("usage: %s <cfg> <weights> <input|-> <batch> <iterations> <nasm file> <output file>\n", argv[0]);
        return 2;
    }
    char *input = strcmp(argv[3], "-") == 0 ? NULL : argv[3];
    const int batch = atoi(argv[4]), iterations = atoi(argv[5]);

    aspen_dnn_t *dnn = apu_create_dnn(argv[1], argv[2]);
    if (dnn == NULL) { ERROR_PRTF("cannot build the dnn from %s\n", argv[1]); return 1; }
    nasm_t *made = apu_create_nasm(dnn, 8, (unsigned)batch);
    if (made == NULL) { ERROR_PRTF("cannot build the nasm\n"); return 1; }
    apu_save_nasm_to_file(made, argv[6]);
    apu_destroy_nasm(made);
    nasm_t *nasm = apu_load_nasm_from_file(argv[6], dnn);
    if (nasm == NULL) { ERROR_PRTF("cannot load %s\n", argv[6]); return 1; }

    rpool_t *rpool = rpool_init();
    dse_group_t *dses = dse_group_init(4);
    if (dses == NULL) { RED_PRTF("no execution engine\n"); return 3; }
    dse_group_set_rpool(dses, rpool);
    rpool_add_nasm(rpool, nasm, input);

    double t0 = now_sec();
    for (int i = 0; i < iterations; i++) {
        rpool_reset_queue(rpool);
        rpool_reset_nasm(rpool, nasm);
        dse_group_run(dses);
        dse_wait_for_nasm_completion(nasm);
        dse_group_stop(dses);
    }
    GREEN_PRTF("%d iterations, %f s each\n", iterations, (now_sec() - t0) / (iterations > 0 ? iterations : 1));
    if (dse_check_nasm_completion(nasm) != 1) { ERROR_PRTF("the graph did not complete\n"); return 4; }

    LAYER_PARAMS order[] = {BATCH, OUT_C, OUT_H, OUT_W};
    void *result = NULL;
    ssize_t bytes = dse_get_nasm_result(nasm, order, &result);
    if (bytes <= 0) { ERROR_PRTF("no result\n"); return 5; }
    FILE *f = fopen(argv[7], "wb");
    if (f == NULL) { ERROR_PRTF("cannot write %s\n", argv[7]); return 6; }
    fwrite(result, (size_t)bytes, 1, f);
    fclose(f);
    free(result);

    dse_group_destroy(dses);
    rpool_destroy(rpool);
    apu_destroy_nasm(nasm);
    apu_destroy_dnn(dnn);
    return 0;
}
