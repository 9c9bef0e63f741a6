/* A C translation unit against include/hl_b200.h, linked to the library: the header is valid C99 (what a cgo / Rust
 * bindgen / JNI binding consumes), every prototype a binding would use is callable with the documented argument types, and,
 * with the argument "gpu", one small hiding commitment with its opening calls runs through the C ABI from plain C.
 *
 *   gcc -std=c99 -Wall -Wextra -Werror -pedantic -Iinclude tests/c_abi/abi_smoke.c -o abi_smoke -Lintelligenceregulation_b200 -lhl_b200
 *
 * Without arguments nothing touches a device: the program takes the address of every entry point through a typed function
 * pointer (a prototype that drifted from this file's expectation fails to compile) and checks the argument refusals that
 * are answered before any CUDA call.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "hl_b200.h"
#include "hl_b200_bench.h"

#define P 0xFFFFFFFF00000001ULL

typedef int (*commit_zk_fn)(hl_ctx*, uint32_t, uint32_t, const uint64_t*, size_t, const uint64_t*, size_t, const uint64_t*, uint32_t, const uint8_t*,
                            hl_store**, uint8_t*);
typedef int (*packed_fn)(hl_ctx*, uint32_t, uint32_t, const void*, const uint8_t*, size_t, const uint64_t*, size_t, const uint64_t*, uint32_t,
                         const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, hl_store**, uint8_t*, uint8_t*);
typedef int (*fold_fn)(hl_store*, const uint64_t*, size_t, int, uint64_t*);
typedef int (*columns_fn)(hl_store*, const uint64_t*, size_t, uint64_t*);
typedef int (*rounds_new_ir_fn)(hl_ctx*, size_t, uint32_t, uint32_t, const uint64_t*, const uint32_t*, size_t, uint32_t, uint32_t, const uint64_t*,
                                size_t, hl_rounds**);
typedef int (*static_hash_fn)(const uint64_t*, size_t, size_t, const uint8_t*, uint8_t*, void*);
typedef int (*verify_fn)(hl_ctx*, const uint64_t*, size_t, size_t, const uint64_t*, const uint8_t*, const uint8_t*, uint32_t, const uint8_t*, const uint8_t*,
                         const uint8_t*, const uint8_t*, const uint64_t*, size_t, const uint64_t*, const hl_store*, int32_t*, int64_t*);

static uint64_t addmod(uint64_t a, uint64_t b) { /* a, b < p */
    uint64_t s = a + b;
    if (s < a || s >= P) s -= P;
    return s;
}
static uint64_t mulmod(uint64_t a, uint64_t b) { /* double and add: the test needs a few hundred products */
    uint64_t r = 0;
    a %= P;
    while (b) {
        if (b & 1) r = addmod(r, a);
        a = addmod(a, a);
        b >>= 1;
    }
    return r;
}

int main(int argc, char** argv) {
    commit_zk_fn f1 = hl_b200_commit_zk;
    packed_fn f2 = hl_b200_commit_zk_packed;
    fold_fn f3 = hl_b200_store_fold;
    columns_fn f4 = hl_b200_store_columns;
    rounds_new_ir_fn f5 = hl_b200_rounds_new_ir;
    static_hash_fn f6 = hl_b200_hash_columns_static;
    verify_fn f7 = hl_b200_verify_columns;
    if (!f1 || !f2 || !f3 || !f4 || !f5 || !f6 || !f7) return 1;
    if (hl_b200_verify_opening(NULL, 4, 2, 4, NULL, NULL, 0, NULL, 0, 0, NULL, NULL, NULL, 0, NULL, NULL, NULL, NULL, NULL, NULL, NULL) != HL_B200_ERR_ARG) return 6;
    if (hl_b200_verify_columns(NULL, NULL, 0, 0, NULL, NULL, NULL, 0, NULL, NULL, NULL, NULL, NULL, 0, NULL, NULL, NULL, NULL) != HL_B200_ERR_ARG) return 5;
    /* refusals that need no device */
    if (hl_b200_store_fold(NULL, NULL, 0, 0, NULL) != HL_B200_ERR_ARG) return 2;
    if (hl_b200_hash_columns_static(NULL, 1, 1, NULL, NULL, NULL) != HL_B200_ERR_ARG) return 3;
    if (hl_b200_rounds_round(NULL, 0, 1, NULL) != HL_B200_ERR_ARG) return 4;
    if (argc < 2 || strcmp(argv[1], "gpu") != 0) {
        printf("abi ok (no device touched)\n");
        return 0;
    }
    /* one hiding commitment of 6 rows x 256 words at rate 1/2 with 8 pads per row, from plain C */
    hl_ctx* ctx = NULL;
    if (hl_b200_init(0, &ctx) != HL_B200_OK) { fprintf(stderr, "init failed\n"); return 10; }
    enum { LOGN = 8, N = 256, NN = 512, ROWS = 6, Q = 8 };
    uint64_t* data = malloc(sizeof(uint64_t) * ROWS * N);
    uint64_t* pads = malloc(sizeof(uint64_t) * ROWS * Q);
    uint64_t* pows = malloc(sizeof(uint64_t) * NN);
    uint8_t* leaves = malloc(32 * NN);
    uint8_t* leaves2 = malloc(32 * NN);
    uint8_t* packed = malloc(2 * ROWS * N);
    uint8_t widths[ROWS];
    for (int i = 0; i < ROWS * N; i++) {  /* int16-valued words: x >= 0 as x, x < 0 as p + x */
        int v = (int)((i * 2654435761u) >> 16) % 65536 - 32768;
        data[i] = v >= 0 ? (uint64_t)v : P - (uint64_t)(-v);
        packed[2 * i] = (uint8_t)(v & 0xFF);
        packed[2 * i + 1] = (uint8_t)((v >> 8) & 0xFF);
    }
    for (int r = 0; r < ROWS; r++) widths[r] = 2;
    for (int i = 0; i < ROWS * Q; i++) pads[i] = mulmod(0x9E3779B97F4A7C15ULL % P, (uint64_t)i + 1);
    pows[0] = 1;
    for (int i = 1; i < NN; i++) pows[i] = mulmod(pows[i - 1], 7);
    hl_store *st = NULL, *st2 = NULL;
    int rc = hl_b200_commit_zk(ctx, LOGN, 2, data, ROWS, pads, Q, pows, LOGN + 1, NULL, &st, leaves);
    if (rc != HL_B200_OK) { fprintf(stderr, "commit_zk: %d %s\n", rc, hl_b200_last_error(ctx)); return 11; }
    rc = hl_b200_commit_zk_packed(ctx, LOGN, 2, packed, widths, ROWS, pads, Q, pows, LOGN + 1, NULL, NULL, NULL, NULL, &st2, leaves2, NULL);
    if (rc != HL_B200_OK) { fprintf(stderr, "commit_zk_packed: %d %s\n", rc, hl_b200_last_error(ctx)); return 12; }
    if (memcmp(leaves, leaves2, 32 * NN) != 0) { fprintf(stderr, "the packed rows commit to other leaves\n"); return 13; }
    /* rho^T [M | pads] with rho = e_2: the fold returns row 2 and its pads */
    uint64_t rho[ROWS * 2];
    memset(rho, 0, sizeof rho);
    rho[2 * 2] = 1;
    uint64_t* out = malloc(sizeof(uint64_t) * (N + Q) * 2);
    rc = hl_b200_store_fold(st2, rho, 1, 1, out);
    if (rc != HL_B200_OK) return 14;
    for (int j = 0; j < N; j++)
        if (out[2 * j] != data[2 * N + j] || out[2 * j + 1] != 0) { fprintf(stderr, "fold word %d\n", j); return 15; }
    for (int j = 0; j < Q; j++)
        if (out[2 * (N + j)] != pads[2 * Q + j]) return 16;
    uint64_t idx[2] = {0, NN - 1};
    uint64_t cols[2 * ROWS], cols2[2 * ROWS];
    if (hl_b200_store_columns(st, idx, 2, cols) != HL_B200_OK || hl_b200_store_columns(st2, idx, 2, cols2) != HL_B200_OK) return 17;
    if (memcmp(cols, cols2, sizeof cols) != 0) return 18;
    hl_stats s;
    if (hl_b200_stats(ctx, &s) != HL_B200_OK || s.commits != 2 || s.declines != 0) return 19;
    hl_b200_store_free(st);
    hl_b200_store_free(st2);
    hl_b200_shutdown(ctx);
    printf("abi ok: %s\n", "two commitments, fold and columns through the C ABI");
    free(data); free(pads); free(pows); free(leaves); free(leaves2); free(packed); free(out);
    return 0;
}
