// Test infrastructure: a minimal host-side stand-in for the CUDA execution model, just large
// enough to run simple `extern "C" __global__` kernels (plain C bodies, optional __shared__
// arrays and __syncthreads) UNCHANGED on the CPU with g++.
//
// It exists so that the CUDA C kernel strings the reference project keeps in
// src/shaders/cuda.rs can be compiled from where they lie and executed here, giving outputs of
// the reference's own kernel code to hold the oracle (akasha_oracle.c) to. `make_ref.py` beside
// this file pastes the strings, read at run time, after an #include of this header; nothing of
// the reference is stored in this repository.
//
// Model: blocks run one after the other on the calling thread. A kernel that never calls
// __syncthreads runs its threads as a plain loop. A kernel that does runs every thread of a
// block as a ucontext fiber; __syncthreads() yields to the scheduler, which resumes the fibers
// round-robin, so every fiber reaches barrier k before any of them continues past it (threads
// that have returned no longer take part, as on the GPU). `__shared__` becomes `static`, which
// is per-block because blocks do not overlap.
#pragma once
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <ucontext.h>

#include <functional>
#include <vector>

struct shim_dim3 {
    unsigned int x, y, z;
};

static shim_dim3 gridDim, blockDim, blockIdx, threadIdx;

#define __global__
#define __device__
#define __host__
#define __shared__ static
#define __forceinline__ inline
#define __restrict__

static inline float __uint_as_float(unsigned int u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline unsigned int __float_as_uint(float f) {
    unsigned int u;
    memcpy(&u, &f, 4);
    return u;
}
static inline float atomicAdd(float* p, float v) {
    float old = *p;
    *p = old + v;
    return old;
}

namespace shim {

struct Fiber {
    ucontext_t ctx;
    shim_dim3 tid;
    bool done;
    char* stack;
};

static ucontext_t g_sched;
static Fiber* g_cur = nullptr;
static const std::function<void()>* g_body = nullptr;

static void fiber_main() {
    (*g_body)();
    g_cur->done = true;
    swapcontext(&g_cur->ctx, &g_sched);
}

static inline void yield_to_scheduler() {
    Fiber* me = g_cur;
    swapcontext(&me->ctx, &g_sched);
}

// Run `body` (one kernel thread) over the whole launch.
static void run(unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz, bool uses_sync,
                const std::function<void()>& body) {
    gridDim = {gx, gy, gz};
    blockDim = {bx, by, bz};
    const size_t nthreads = (size_t)bx * by * bz;
    const size_t STACK = 256 * 1024;   // the flash kernel keeps float acc[128] on its stack
    std::vector<Fiber> fibers;
    std::vector<char> stacks;
    if (uses_sync) {
        fibers.resize(nthreads);
        stacks.resize(nthreads * STACK);
    }
    for (unsigned z = 0; z < gz; z++)
        for (unsigned y = 0; y < gy; y++)
            for (unsigned x = 0; x < gx; x++) {
                blockIdx = {x, y, z};
                if (!uses_sync) {
                    for (unsigned tz = 0; tz < bz; tz++)
                        for (unsigned ty = 0; ty < by; ty++)
                            for (unsigned tx = 0; tx < bx; tx++) {
                                threadIdx = {tx, ty, tz};
                                body();
                            }
                    continue;
                }
                g_body = &body;
                size_t i = 0;
                for (unsigned tz = 0; tz < bz; tz++)
                    for (unsigned ty = 0; ty < by; ty++)
                        for (unsigned tx = 0; tx < bx; tx++, i++) {
                            Fiber& f = fibers[i];
                            f.tid = {tx, ty, tz};
                            f.done = false;
                            f.stack = stacks.data() + i * STACK;
                            getcontext(&f.ctx);
                            f.ctx.uc_stack.ss_sp = f.stack;
                            f.ctx.uc_stack.ss_size = STACK;
                            f.ctx.uc_link = &g_sched;
                            makecontext(&f.ctx, fiber_main, 0);
                        }
                size_t live = nthreads;
                while (live) {
                    live = 0;
                    for (size_t k = 0; k < nthreads; k++) {
                        Fiber& f = fibers[k];
                        if (f.done) continue;
                        g_cur = &f;
                        threadIdx = f.tid;
                        swapcontext(&g_sched, &f.ctx);
                        if (!f.done) live++;
                    }
                }
            }
}

}  // namespace shim

static inline void __syncthreads() { shim::yield_to_scheduler(); }
