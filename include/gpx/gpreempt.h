// set_priority / NvRmQuery with the reference's names (include/gpreempt.h:111-173,
// src/gpreempt.cpp:33-72).  The reference finds the calling thread's channel group with an ioctl
// of a patched driver and sets its timeslice (1 s for priority 0, 1 us for priority 1).  No
// driver setting is touched here: the priority class selects the CUDA stream priority of streams
// this thread creates afterwards, and preemption itself happens inside the kernels.
#pragma once

#include "../gpx.h"

typedef unsigned int NvHandle;
typedef unsigned int NV_STATUS;
#define NV_OK 0u

struct NvChannels {
    unsigned int numChannels = 0;
};

struct NvContext {
    NvHandle hClient = 0;
    NvHandle hObject = 0;
    NvChannels channels;
};

// NvRmQuery, src/gpreempt.cpp:33-50: nothing to look up without the driver escape.
inline NV_STATUS NvRmQuery(NvContext *pContext) { return pContext ? NV_OK : 1u; }

// set_priority, src/gpreempt.cpp:61-72: 0 = high priority, 1 = low priority.
inline int set_priority(NvContext /*ctx*/, int priority) { return gpx_set_priority(priority); }
