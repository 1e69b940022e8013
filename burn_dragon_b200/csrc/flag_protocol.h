// Arithmetic of the cross-rank flag barrier, shared by the device code (collectives.cu) and by the
// host-side simulation that stress-tests the protocol with real threads (host/hostlib.cpp).
//
// Every rank owns a flag array; slot (cta, writer) of rank r's array is written only by `writer`'s
// CTA `cta` and read only by rank r's CTA `cta`. A barrier with value v: store-release v into my
// slot of every rank's array, then wait (load-acquire) until every slot of my own array has
// reached v. Values only grow: call number `epoch` uses 2*epoch + 1 for the barrier that opens a
// collective and 2*epoch + 2 for the one that closes it, in 32-bit arithmetic, and "reached" is a
// signed distance so the comparison survives the wrap of the 32-bit counter.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define BDH_HD __host__ __device__ __forceinline__
#else
#define BDH_HD inline
#endif

BDH_HD int flag_slot(int cta, int world, int writer) { return cta * world + writer; }
BDH_HD uint32_t flag_value(uint32_t epoch, uint32_t phase) { return 2u * epoch + phase; }   // phase 1 or 2
BDH_HD bool flag_reached(uint32_t seen, uint32_t value) { return static_cast<int32_t>(seen - value) >= 0; }
