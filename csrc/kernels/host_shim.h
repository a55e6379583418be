// Kernel-on-CPU shim: lets the collective kernel bodies (dev_comm.cuh, reduce_ops.cuh, coll_bodies*.cuh) compile as
// plain C++ and run with every CUDA thread as a host thread, so that ThreadSanitizer and AddressSanitizer can watch
// the flag protocols (compute-sanitizer's racecheck cannot see accesses from other GPUs, and is not always available).
//
// The role of the reference's kernel unit-test stub (test/ut/all_reduce_aiv/stub/aiv_communication_base_v2.h:18-125),
// which compiles the production kernel header against a base class that records copies, flag records and flag waits
// per (rank, block) and checks that they resolve.  Here the production code itself runs: data accesses stay plain
// loads and stores (a missing fence or flag shows up as a data race), flags and flag-in-data lines become atomics
// with the memory order the PTX has (st.release.sys -> release, ld.acquire.sys -> acquire, volatile -> relaxed), the
// multimem instructions become loops over the ranks' copies, and every wait is bounded exactly as on the GPU, so a
// protocol that cannot make progress ends with the wait's failure record instead of a hang.
//
// Only included when HCCL_HOST_SHIM is defined (g++ -DHCCL_HOST_SHIM); nvcc never sees it.
#pragma once
#ifdef HCCL_HOST_SHIM
#include <pthread.h>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <vector>
#include <cuda_runtime.h>      // vector types and the no-op meaning of __device__ / __forceinline__ for a host compiler

namespace hostshim {

struct Dim3 { unsigned x = 0, y = 0, z = 0; };
struct BlockCtx {
    pthread_barrier_t bar;
    alignas(16) char shared[64 * 64];      // 64 slots of 64 bytes for HCCL_SHARED variables
};
struct ThreadCtx {
    Dim3 tid, bid, bdim, gdim;
    BlockCtx* block = nullptr;
};
inline ThreadCtx& Tls()
{
    static thread_local ThreadCtx t;
    return t;
}
inline void SyncThreads() { pthread_barrier_wait(&Tls().block->bar); }
template <class T>
inline T* SharedSlot(int id)
{
    static_assert(sizeof(T) <= 64, "HCCL_SHARED slot too small");
    return reinterpret_cast<T*>(Tls().block->shared + (id % 64) * 64);
}
inline uint64_t NowNs()
{
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Multicast aliases: an address inside [mcBase, mcBase + mcBytes) stands for the same offset in every rank's buffer.
struct McWindow { const char* base; size_t bytes; std::vector<char*> targets; };
inline std::vector<McWindow>& McWindows()
{
    static std::vector<McWindow> w;
    return w;
}
inline const McWindow* McFind(const void* p, size_t* off)
{
    for (const McWindow& w : McWindows()) {
        if ((const char*)p >= w.base && (const char*)p < w.base + w.bytes) { *off = (size_t)((const char*)p - w.base); return &w; }
    }
    return nullptr;
}

}  // namespace hostshim

#ifndef __noinline__
#define __noinline__ __attribute__((noinline))
#endif
#define threadIdx (hostshim::Tls().tid)
#define blockIdx (hostshim::Tls().bid)
#define blockDim (hostshim::Tls().bdim)
#define gridDim (hostshim::Tls().gdim)
#define __syncthreads() hostshim::SyncThreads()
#define HCCL_SHARED(T, name) T& name = *hostshim::SharedSlot<T>(__COUNTER__)

inline void __threadfence() { std::atomic_thread_fence(std::memory_order_seq_cst); }
inline void __threadfence_system() { std::atomic_thread_fence(std::memory_order_seq_cst); }
template <class T>
inline T __ldg(const T* p) { return *p; }
inline unsigned atomicCAS(unsigned* p, unsigned cmp, unsigned val)
{
    __atomic_compare_exchange_n(p, &cmp, val, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
    return cmp;
}
inline unsigned long long atomicAdd(unsigned long long* p, unsigned long long v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
inline unsigned atomicAdd(unsigned* p, unsigned v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
inline unsigned long long atomicMax(unsigned long long* p, unsigned long long v)
{
    unsigned long long cur = __atomic_load_n(p, __ATOMIC_RELAXED);
    while (cur < v && !__atomic_compare_exchange_n(p, &cur, v, true, __ATOMIC_SEQ_CST, __ATOMIC_RELAXED)) {}
    return cur;
}
#include <sched.h>
#define HCCL_SPIN_PAUSE() sched_yield()      // far more threads than cores: a waiting thread gives its core away
#else
#define HCCL_SHARED(T, name) __shared__ T name
#define HCCL_SPIN_PAUSE()
#endif
