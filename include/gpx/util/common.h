// Status codes and checking macros with the names client code of thustorage/GPreempt uses
// (include/util/common.h:7-61), for sources that are compiled against libgpx instead.
// No logging library is needed: messages go to stderr.
#pragma once

#include <cstdio>
#include <cstdlib>
#include <exception>
#include <iostream>

#include "../../gpx.h"

#define div_ceil(a, b) (((a) + (b) - 1) / (b))

// include/util/common.h:16-23; numerically equal to enum gpx_status.
enum Status { Succ = GPX_SUCC, Fail = GPX_FAIL, Timeout = GPX_TIMEOUT, NotFound = GPX_NOT_FOUND,
              OutOfRange = GPX_OUT_OF_RANGE, Full = GPX_FULL };

// include/util/common.h:7-14: a failed status ends the program.
#define CHECK_STATUS(cmd)                                                                          \
    {                                                                                              \
        Status s__ = (Status)(cmd);                                                                \
        if (s__ != Status::Succ) {                                                                 \
            std::fprintf(stderr, "%s error (%s: %s), %s:%d\n", #cmd, gpx_strerror((int)s__),      \
                         gpx_last_error(), __FILE__, __LINE__);                                    \
            std::exit(1);                                                                          \
        }                                                                                          \
    }

// include/util/common.h:26-34: the reference terminates before it returns; so does this.
#define RETURN_STATUS(cmd)                                                                         \
    {                                                                                              \
        Status s__ = (Status)(cmd);                                                                \
        if (s__ != Status::Succ) {                                                                 \
            std::fprintf(stderr, "%s error (%s: %s), %s:%d\n", #cmd, gpx_strerror((int)s__),      \
                         gpx_last_error(), __FILE__, __LINE__);                                    \
            std::terminate();                                                                      \
            return s__;                                                                            \
        }                                                                                          \
    }

#define ASSERT(condition)                                                                          \
    do {                                                                                           \
        if (!(condition)) {                                                                        \
            std::cerr << "Assertion `" #condition "` failed in " << __FILE__ << ":" << __LINE__    \
                      << std::endl;                                                                \
            std::terminate();                                                                      \
        }                                                                                          \
    } while (false)

template <typename T>
T align_up(T value, T alignment) {
    T rest = value % alignment;
    return rest == 0 ? value : value - rest + alignment;
}

template <typename T>
T align_down(T value, T alignment) {
    return value - value % alignment;
}

// src/util/util.cpp:3-11.
inline void bind_core(int core_id) {
    if (gpx_bind_core(core_id) != GPX_SUCC) std::fprintf(stderr, "Failed to bind core %d\n", core_id);
}
