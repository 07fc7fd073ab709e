// Tuning knobs of the library, read from the FDA_* environment once per process (first use) instead of
// on every launch; fda_reload_config() re-reads them (tests change them between calls).
#pragma once

namespace fda {

struct Config {
    double l2_keep_fraction;  // FDA_L2_KEEP_FRACTION  share of L2 that may be marked "evict last" (0.7)
    int binning;              // FDA_BINNING           0 switches the slab-binned backward off (1)
    double bin_slab_mb;       // FDA_BIN_SLAB_MB       bytes of the fp32 image per slab or brick, in MB (4)
    int bin_grid_x;           // FDA_BIN_GRID_X        blocks striding over one slab's list (0 = from the entry count)
    int pair_rows;            // FDA_PAIR_ROWS         0 switches the paired-row scatter off (1)
    int forced_variant;       // FDA_FORCE_VARIANT     0 library's choice, 1 "reg", 2 "smem" (forward staging)
    int peer_reduce_blocks;   // FDA_PEER_REDUCE_BLOCKS  blocks of the cross-GPU exchange kernels (32)
    int fwd_head_groups;      // FDA_FWD_HEAD_GROUPS   forward walks the rows head group by head group: 0 never, 1 for large calls whose value volume exceeds L2, 2 whenever the volume exceeds the budget (1)
    int sorted;               // FDA_BWD_SORT          cell-sorted backward: 0 off, 1 for large, dense problems, 2 whenever the shape allows (1)
    int sort_seg;             // FDA_SORT_SEGMENT      list entries per lane group between flushes (32)
    int sort_grid_x;          // FDA_SORT_GRID_X       blocks per batch element walking the sorted list (0 = fill the SMs once)
    int touched;              // FDA_BWD_TOUCHED       fda_backward zero-fills / converts only the image rows the points touch: 0 never, 1 when they can touch at most 60 % of it, 2 always (1)
    int sort_ahead;           // FDA_SORT_AHEAD        points whose rows are in flight per lane of the walk: 2, 3 or 4 (2)
};

const Config &config();

// Remember a failing cudaError_t for fda_last_cuda_error() (per calling thread).
void record_cuda_error(int cuda_error);

}  // namespace fda
