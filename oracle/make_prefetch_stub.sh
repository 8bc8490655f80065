#!/bin/sh
# TEST INFRASTRUCTURE ONLY.  Writes the two headers the upstream platform probe would print
# (pre/prefetch_probe.cu:62-106) for a B200, so that the upstream host code compiles without a GPU.
# Kernel rows: {threads, registers (ptxas -v, sm_100a, nvcc 12.9), static shared bytes,
# iteration_bytes = tasks*(BM*BN + BN*columns)*sizeof(value)}; order 8/32, 8/64, 16/32, 16/64, 64/32, 64/64.
set -e
out="$1"
common='#pragma once
#include <cuda_runtime.h>
struct PrefetchDeviceInfo { int major, minor, sm_count, threads_per_sm; size_t shared_bytes_per_sm; int blocks_per_sm, registers_per_sm, l2_bytes; };
struct PrefetchKernelInfo { int threads, registers_per_thread; size_t shared_bytes; int iteration_bytes; };
static const PrefetchDeviceInfo prefetch_device_info = {10, 0, 148, 2048, 233472, 32, 65536, 132644864};
static inline bool prefetch_device_matches(const cudaDeviceProp &prop) { return prop.major == prefetch_device_info.major && prop.minor == prefetch_device_info.minor; }
'
{
printf '%s' "$common"
cat <<'EOT'
static const PrefetchKernelInfo prefetch_kernel_info[6] = {
    {128, 46, 5120, 5120}, {64, 42, 2304, 2304}, {128, 46, 10240, 6144}, {64, 40, 4608, 2560},
    {128, 40, 5120, 6144}, {256, 40, 9216, 8192},
};
EOT
} > "$out/prefetch_fp16.h"
{
printf '%s' "$common"
cat <<'EOT'
static const PrefetchKernelInfo prefetch_kernel_info[6] = {
    {128, 52, 5120, 5120}, {64, 42, 2304, 2304}, {128, 48, 10240, 6144}, {64, 40, 4608, 2560},
    {128, 46, 5120, 6144}, {256, 54, 9216, 8192},
};
EOT
} > "$out/prefetch_tf32.h"
