// Process-wide switches of the library, for A/B measurements and for tests that push one input
// through every kernel family.  Read from the environment ONCE, at first use; changed afterwards
// only through sbnet_set_option() (include/sbnet_b200.h).  Plain ints: a change made while another
// thread is launching is seen by that launch or by the next one.
#pragma once

namespace sbnet {

struct Options {
    int planes;        // plane-layout dispatch: 0 default, 1 persistent TMA pipeline, 2 tile CTAs with plain loads
                       //   (SBNET_PLANES=tma|tile), 3 tile CTAs fed by TMA whatever the launch size,
                       //   4 general shapes run the element-wise (planes) / narrow-vector (rows) kernels instead of
                       //   the raw-row kernel,
                       //   6 the raw-row kernel with element-wide (never vector) accesses on the stack side
    int disableTma;    // 1: plane layouts run the general kernel only (SBNET_DISABLE_TMA=1)
    int tileBlocks;    // > 0: blocks per shared tile regardless of the launch size (SBNET_TILE_BLOCKS)
    int rmKernel;      // reduce_mask: 0 default, 1 band kernel, 2 one thread per block (SBNET_RM_KERNEL)
    int rmCtasPerSm;   // reduce_mask tile kernel: CTAs per SM the column tiling aims at (SBNET_RM_CTAS_PER_SM)
    int rmResident;    // reduce_mask tile kernel: at most this many CTAs resident per SM, 0 = no cap (SBNET_RM_RESIDENT)
    int pdl;           // launch every kernel with programmatic stream serialization (SBNET_PDL, default 1)
    int tmaL2;         // L2 promotion of the image tensor maps: 0 none, 1 64 B, 2 128 B, 3 256 B (SBNET_TMA_L2, default 3)
};

Options& options();

} // namespace sbnet
