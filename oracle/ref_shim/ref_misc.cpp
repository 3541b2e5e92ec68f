// Thread count and deallocation for the reference-CPU checker library.
#include <cstdlib>

#include "ref_abi.h"
#include "tbb/info.h"

extern "C" int ref_threads(void) { return tbb::info::default_concurrency(); }
extern "C" void ref_free(void *p) { std::free(p); }
