// Timeline probe for timing studies: a few device-wide timestamps per kernel launch, kept with
// atomics so that they hold the earliest start and the latest of each later event over all CTAs.
//   [0] first CTA started   [1] last CTA passed its dependency wait
//   [2] last CTA finished its prologue   [3] last warp finished
//   [4] last CTA started   [5] last CTA finished its set-up (before the dependency wait); 8 words per launch
// A null pointer (the normal case) costs one predictable branch per event.
#pragma once
#include <cstdint>

namespace tlb {

__device__ __forceinline__ unsigned long long span_now()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void span_start(unsigned long long *span)
{
    if (span) atomicMin(span, span_now());
}
__device__ __forceinline__ void span_event(unsigned long long *span, int which)
{
    if (span) atomicMax(span + which, span_now());
}

}  // namespace tlb
