// SSD-MIMO chunked scan, precision "io": bf16 operands on tcgen05 tensor cores (placeholder until the tiles land).
#include "common.cuh"
#include "scan_args.h"

namespace orbit {
int tc_supported(const ScanArgs&, int, const char** why) { *why = "tensor-core tiles not built yet"; return 0; }
int tc_pick_chunk(int, int, int, int, int, int) { return 0; }   // 0: geometry not served by the tensor-core tiles
int tc_launch_chunk_state(const ScanArgs&, cudaStream_t) { return fail(ERR_UNSUPPORTED, "precision 'io' not built"); }
int tc_launch_chunk_out(const ScanArgs&, cudaStream_t) { return fail(ERR_UNSUPPORTED, "precision 'io' not built"); }
int tc_launch_chunk_dstate(const ScanArgs&, cudaStream_t) { return fail(ERR_UNSUPPORTED, "precision 'io' not built"); }
int tc_launch_chunk_grads(const ScanArgs&, cudaStream_t) { return fail(ERR_UNSUPPORTED, "precision 'io' not built"); }
}  // namespace orbit
