/* Stand-in for <glog/logging.h>, which the reference's headers include but this image lacks.
 * Only the streaming form LOG(level) << ... is used there (include/util/gpu_util.h:148,
 * include/util/common.h:11,30); it goes to stderr.  Test infrastructure: used solely to compile
 * the reference's miniWeather source, unmodified, into oracle/_ref. */
#pragma once
/* glog's header brings these standard headers with it, and the reference's headers rely on that. */
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <memory>
#include <set>
#include <sstream>
#include <string>
#include <vector>
#define LOG(level) (std::cerr << "[" #level "] ")
