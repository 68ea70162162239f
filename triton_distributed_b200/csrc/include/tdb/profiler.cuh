// Intra-kernel profiler: a kernel records (tag, globaltimer) pairs into a pre-allocated 64-bit buffer; the host turns
// them into a Chrome / Perfetto trace with one track per (SM, group).
//
// Record layout (64 bits): [63:44] block id  [43:33] group  [32:22] task type  [21] start flag ... no: kept simple:
//   word = (tag << 32) | globaltimer_lo, tag = block(16) | group(4) | task(11) | is_start(1)
// Buffer layout: slot 0 = number of records written (atomic counter), slot 1 = capacity, then per record 2 words:
//   {tag | time_lo, smid}.
// Matches the reference's tools/profiler/language.py:84-172 (Profiler.create / record) in purpose.
#pragma once
#include "ptx.cuh"

namespace tdb {

struct ProfilerBuf {
  unsigned long long* buf;   // nullptr = profiling off
};

TDB_DEVICE void profile_record(const ProfilerBuf& p, uint32_t group, uint32_t task, bool is_start) {
  if (p.buf == nullptr) return;
  const unsigned long long cap = p.buf[1];
  const unsigned long long idx = atomicAdd(p.buf, 1ull);
  if (idx >= cap) return;
  const uint32_t tag = ((blockIdx.x & 0xffffu) << 16) | ((group & 0xfu) << 12) | ((task & 0x7ffu) << 1) | (is_start ? 1u : 0u);
  const unsigned long long t = globaltimer_ns();
  p.buf[2 + 2 * idx] = (static_cast<unsigned long long>(tag) << 32) | (t & 0xffffffffull);
  p.buf[3 + 2 * idx] = (static_cast<unsigned long long>(sm_id()) << 32) | (t >> 32);
}

#define TDB_PROFILE_RECORD(prof, group, task, is_start) \
  do {                                                  \
    if (threadIdx.x % 32 == 0) ::tdb::profile_record((prof), (group), (task), (is_start)); \
  } while (0)

}  // namespace tdb
