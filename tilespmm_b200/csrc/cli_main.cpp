// tilespmm_fp16 / tilespmm_tf32 -d <device_id> <matrix.mtx> <colB> [--gpus N]
//
// Drop-in for the two upstream executables (src/main.cu:136-352): same arguments and exit codes, the same
// synthetic inputs (srand(1325), values 1 + rand() % 3 in CSR order, then B, src/main.cu:177-207), the same 19-field
// CSV row without header appended to TileSpMM-FP16.csv / TileSpMM-TF32.csv in the working directory
// (src/main.cu:293-308, src/csr2tile.h:1062, src/main.cu:82,115), the same check against cuSPARSE at 1e-3 absolute
// (src/main.cu:315-335).  Everything on the GPU goes through the C ABI of libtilespmm_b200.so.
// Opt-in extension, absent upstream: a trailing `--gpus N` spreads the panels of A over the devices device_id ..
// device_id+N-1 (tsp_multi_*); the CSV row keeps its 19 fields (thresholds of the first device, time of the slowest).
// Built once per precision with -DTSP_PRECISION=0 (FP16) or 1 (TF32).
#include <cuda_runtime.h>
#include <limits.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include "../../include/tilespmm_b200.h"

#ifndef TSP_PRECISION
#define TSP_PRECISION 0
#endif
#ifndef BENCH_REPEAT
#define BENCH_REPEAT 1000
#endif
#ifndef WARMUP_NUM
#define WARMUP_NUM 100
#endif

extern "C" int tsp_read_mtx(const char *path, int *m, int *n, long long *nnz, int *is_symmetric, int **h_rowptr, int **h_colidx, float **h_val);
extern "C" void tsp_free_host(void *p);

static uint16_t half_bits(float f)  // float -> binary16, round to nearest even
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t man = x & 0x7fffffu;
    if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0)
    {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const int shift = 14 - exp;
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (h & 1))) h++;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;
    return (uint16_t)(sign | h);
}

static double wall_ms()
{
    struct timeval t;
    gettimeofday(&t, NULL);
    return t.tv_sec * 1000.0 + t.tv_usec / 1000.0;
}

#define FAIL_IF(rc, what)                                                      \
    do {                                                                       \
        if (rc) { fprintf(stderr, "%s: %s\n", what, tsp_last_error()); return EXIT_FAILURE; } \
    } while (0)

int main(int argc, char **argv)
{
    if (argc < 5 || strcmp(argv[1], "-d") != 0)
    {
        printf("Usage: %s -d device_id matrix.mtx colB\n", argv[0]);
        return EXIT_FAILURE;
    }
    int gpus = 1;
    for (int a = 5; a + 1 < argc; a++)
        if (strcmp(argv[a], "--gpus") == 0) gpus = atoi(argv[a + 1]);
    if (gpus < 1 || gpus > 64) { fprintf(stderr, "--gpus must be between 1 and 64.\n"); return EXIT_FAILURE; }
    printf("--------------------------------!!!!!!!!------------------------------------\n");
    const int device_id = atoi(argv[2]);
    printf("device_id = %i\n", device_id);
    char *filename = argv[3];
    printf("MAT: -------------- %s --------------\n", filename);
    int rowA = 0, colA = 0, is_symmetric = 0, *rowptr = NULL, *colidx = NULL;
    long long nnz64 = 0;
    float *file_val = NULL;
    double t1 = wall_ms();
    FAIL_IF(tsp_read_mtx(filename, &rowA, &colA, &nnz64, &is_symmetric, &rowptr, &colidx, &file_val), "load matrix");
    const int nnzA = (int)nnz64;
    printf("  input matrix A: ( %i, %i ) nnz = %i\n  loadfile time    = %4.5f sec\n", rowA, colA, nnzA, (wall_ms() - t1) / 1000.0);
    const int colB = atoi(argv[4]);
    if (colB <= 0 || colB > INT_MAX - 63)
    {
        fprintf(stderr, "colB must be positive and fit the padded kernel width.\n");
        return EXIT_FAILURE;
    }
    const int colB_padded = colB <= 32 ? 32 : ((colB + 63) / 64) * 64;
    printf("  colB = %d, padded colB = %d\n", colB, colB_padded);

    // the values in the file are replaced by a reproducible integer stream, exactly like upstream
    const size_t vsz = TSP_PRECISION ? 4 : 2;
    srand(1325);
    void *valA = malloc((size_t)(nnzA ? nnzA : 1) * vsz);
    for (int i = 0; i < nnzA; i++)
    {
        const float v = (float)(1 + rand() % 3);
        if (TSP_PRECISION) ((float *)valA)[i] = v; else ((uint16_t *)valA)[i] = half_bits(v);
    }
    tsp_free_host(file_val);
    const size_t b_elems = (size_t)colA * (size_t)colB_padded;
    void *matrixB = malloc(b_elems * vsz);
    if (!valA || !matrixB) { fprintf(stderr, "Host memory allocation failed\n"); return EXIT_FAILURE; }
    for (int row = 0; row < colA; row++)
        for (int col = 0; col < colB_padded; col++)
        {
            const size_t i = (size_t)row * colB_padded + col;
            const float v = col < colB ? (float)(1 + rand() % 3) : 0.0f;
            if (TSP_PRECISION) ((float *)matrixB)[i] = v; else ((uint16_t *)matrixB)[i] = half_bits(v);
        }

    cudaDeviceProp prop;
    if (cudaSetDevice(device_id) != cudaSuccess || cudaGetDeviceProperties(&prop, device_id) != cudaSuccess)
    {
        fprintf(stderr, "CUDA error select device: %s\n", cudaGetErrorString(cudaGetLastError()));
        return EXIT_FAILURE;
    }
    int clock_khz = 0;
    cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, device_id);
    printf("---------------------------------------------------------------------------------------------\n");
    printf("  Device [ %i ] %s @ %4.2f MHz\n", device_id, prop.name, clock_khz * 1e-3f);

    tsp_handle *h = NULL;
    tsp_multi *mg = NULL;
    if (gpus > 1)
    {
        int devices[64];
        for (int i = 0; i < gpus; i++) devices[i] = device_id + i;
        FAIL_IF(tsp_multi_create(&mg, gpus, devices, TSP_PRECISION), "create");
        printf("  panels of A spread over %d devices (%d..%d)\n", gpus, device_id, device_id + gpus - 1);
    }
    else FAIL_IF(tsp_create(&h, device_id, TSP_PRECISION), "create");
    t1 = wall_ms();
    double features[11];
    const double capability = prop.major + prop.minor / 10.0;
    if (!tsp_features_from_csr(rowA, colA, nnzA, rowptr, capability, colB, features))
    {
        fprintf(stderr, "Cannot extract model features from the input CSR matrix.\n");
        return EXIT_FAILURE;
    }
    float gamma = 0.0f, delta = 0.0f;
    if (TSP_PRECISION) tilespmm_predict_tf32(features, &gamma, &delta); else tilespmm_predict_fp16(features, &gamma, &delta);
    if (mg) FAIL_IF(tsp_multi_convert_host(mg, rowA, colA, nnzA, rowptr, colidx, valA, gamma, delta), "convert");
    else FAIL_IF(tsp_convert_host(h, rowA, colA, nnzA, rowptr, colidx, valA, gamma, delta, 0, 1), "convert");
    const double pre_time = wall_ms() - t1;
    printf("  CPU preprocessing time = %4.5f s\n", pre_time / 1000.0);
    int info[12];
    if (mg) tsp_multi_info(mg, info, NULL); else tsp_info(h, info, NULL);

    const char *csv_path = TSP_PRECISION ? "TileSpMM-TF32.csv" : "TileSpMM-FP16.csv";
    FILE *fout = fopen(csv_path, "a");
    if (fout == NULL) { printf("Writing results fails.\n"); return EXIT_FAILURE; }
    fprintf(fout, "%s,%d,%d,%d,%d,%d,%d,%d,%.1f,%.1f,", filename, rowA, colA, nnzA, colB, info[3], info[7], info[11], gamma, delta);
    fflush(fout);

    float *matrixC = (float *)malloc(sizeof(float) * (size_t)rowA * colB_padded);
    float *matrixC_cusparse = (float *)malloc(sizeof(float) * (size_t)rowA * colB);
    if (!matrixC || !matrixC_cusparse) { fprintf(stderr, "Host memory allocation failed\n"); return EXIT_FAILURE; }
    double out6[6], out3[3];
    if (mg) FAIL_IF(tsp_multi_run(mg, matrixB, matrixC, colB_padded, colB, pre_time, BENCH_REPEAT, out6), "run");
    else FAIL_IF(tsp_run(h, matrixB, matrixC, colB_padded, colB, pre_time, BENCH_REPEAT, out6), "run");
    printf("  TileSpMM runtime %4.3f ms, %4.3f TFlops\n", out6[4], out6[5]);
    fprintf(fout, "%d,%d,%d,%.9g,%.9g,%.9g,", (int)out6[0], (int)out6[1], (int)out6[2], out6[3], out6[4], out6[5]);
    fflush(fout);

    int rc = tsp_cusparse_baseline(device_id, TSP_PRECISION, rowA, colA, nnzA, rowptr, colidx, valA, colB, colB_padded, matrixB,
                                   matrixC_cusparse, WARMUP_NUM, BENCH_REPEAT, out3);
    FAIL_IF(rc, "cusparse");
    fprintf(fout, "%.9g,", out3[0]);
    printf("  cuSPARSE runtime %4.3f ms, %4.3f Tflops\n", out3[1], out3[2]);
    fprintf(fout, "%.9g,%.9g\n", out3[1], out3[2]);
    fflush(fout);

    size_t errors = 0;
    for (int row = 0; row < rowA; row++)
        for (int col = 0; col < colB; col++)
        {
            const double a = (double)matrixC[(size_t)row * colB_padded + col], b = (double)matrixC_cusparse[(size_t)row * colB + col];
            if (!isfinite(a) || !isfinite(b) || fabs(b - a) > 1e-3)
            {
                if (errors < 10) printf("  c[%d][%d], tilespmm: %lf, cusparse: %lf\n", row, col, a, b);
                errors++;
            }
        }
    if (errors == 0) printf("  Check... PASS!\n");
    else printf("  Check... NO PASS! error_count_cuda = %zu\n", errors);
    fclose(fout);
    tsp_destroy(h);
    tsp_multi_destroy(mg);
    free(matrixC); free(matrixC_cusparse); free(matrixB); free(valA);
    tsp_free_host(rowptr); tsp_free_host(colidx);
    return EXIT_SUCCESS;
}
