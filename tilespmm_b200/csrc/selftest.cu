// Failure-path self test: a kernel whose bounded wait is certain to run out, without hanging or faulting anything.
//
// Every wait inside the tcgen05 kernels of this library (on an mbarrier that a copy, an MMA commit or another warp
// completes) is bounded: after a fixed number of polls the kernel records a code in the handle's device flag, drains
// what it has in flight, frees its tensor memory and returns; the host turns the flag into TSP_ETIMEOUT.  In normal
// operation no wait runs out, so that path would never execute.  This kernel executes it on purpose: it allocates
// tensor memory like the real kernels, initialises an mbarrier that nobody ever arrives on, polls it `polls` times
// with the same try_wait loop, gives up, sets the flag, frees the tensor memory and returns.  Upstream has no
// counterpart (its kernels have no waits and its host code exits on any CUDA error, src/common.h:84-94).
#include "tsp_internal.cuh"

namespace
{

__global__ void __launch_bounds__(64) k_selftest_wait(unsigned polls, int *__restrict__ err)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ unsigned tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned bar_s = (unsigned)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0)
    {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar_s), "r"(1u));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(&tmem_slot)), "r"(32) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_slot;
    if (warp == 0 && lane == 0)
    {
        bool done = false;
        for (unsigned it = 0; it < polls && !done; it++)   // the bounded wait of the real kernels, with a caller-chosen bound
        {
            unsigned p;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                         : "=r"(p) : "r"(bar_s), "r"(0u) : "memory");
            done = p != 0;
        }
        if (!done) atomicExch(err, 0x10);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1)
    {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(32) : "memory");
    }
}

}  // namespace

int tsp_launch_selftest_wait(tsp_handle *h, unsigned polls, cudaStream_t s)
{
    k_selftest_wait<<<1, 64, 0, s>>>(polls, h->d_error);
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}
