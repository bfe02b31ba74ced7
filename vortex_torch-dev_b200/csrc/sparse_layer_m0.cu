// One-launch sparse layer, score mode 0: group mean . centroid scores (block_sparse_attention).
#include "sparse_layer_kernel.cuh"

namespace vtx {
int launch_sparse_layer_m0(const vtxidx::IndexerArgs& ia, const vtxdec::DecodeArgs& da, const vtxidx::AppendArgs& ap, int eff_bs,
                            int group, bool early, cudaStream_t st) {
    switch (ia.D) {
        case 64: return launch_sparse_layer_d<64, 0>(ia, da, ap, eff_bs, group, early, st);
        case 128: return launch_sparse_layer_d<128, 0>(ia, da, ap, eff_bs, group, early, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}
}  // namespace vtx
