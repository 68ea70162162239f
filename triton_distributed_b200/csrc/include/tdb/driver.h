// Run-time lookup of CUDA driver entry points (the library never links libcuda).
#pragma once
#include <cuda.h>

namespace tdb {

// Returns nullptr when the symbol (or a driver) is not available.
void* driver_entry(const char* name);

#define TDB_DRIVER_FN(name) reinterpret_cast<decltype(&name)>(::tdb::driver_entry(#name))

}  // namespace tdb
