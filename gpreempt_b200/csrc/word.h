// The preempt word: one 32-bit flag per GPU that every preemptible kernel polls.  Counterpart
// of the GDRCopy-mapped GdrEntry of the reference (src/cuda-clients/blpclient.cpp:30-76).
#pragma once

#include "common.h"

struct gpx_word {
    int transport;
    int *host_alias;       // pinned host word (MAPPED) or host shadow of the value (DEVICE)
    int *dptr;             // address kernels poll
    cudaStream_t wstream;  // DEVICE transport: dedicated highest-priority stream for the writes
    int device;
};
