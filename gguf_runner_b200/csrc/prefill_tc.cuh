// placeholder
#pragma once
#include <string>
#include "common.cuh"
namespace ggr {
struct PrefillTcArgs { KvView kv; Visibility vis; int layer, seq, base_pos, m; const __nv_bfloat16* q; float* out; float score_scale; };
inline bool prefill_tc_usable(int, int, int, int) { return false; }
inline int launch_prefill_tc(const PrefillTcArgs&, int, int, int, cudaStream_t, std::string* msg) { *msg = "not built"; return 5; }
}
