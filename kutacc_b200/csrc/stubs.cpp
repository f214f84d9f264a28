// Entry points of the reference that lie outside the gated-attention path. They are exported so
// that a program linked against the reference library still resolves its symbols; calling one
// reports an error through the usual convention and returns.
// (include/kutacc.h:266,277,367,379,388 of the reference.)
#include "common.h"

#define KUTACC_NOT_BUILT(name)                                                              \
    extern "C" KUTACC_B200_API void name(void)                                              \
    {                                                                                       \
        KUTACC_CHECK(false, #name ": not part of the B200 gated-attention build");         \
    }

KUTACC_NOT_BUILT(kutacc_af2_outer_product_mean_calc_left_and_right_mul)
KUTACC_NOT_BUILT(kutacc_af2_outer_product_mean_chunk)
KUTACC_NOT_BUILT(kutacc_af2_invariant_point)
KUTACC_NOT_BUILT(kutacc_af2_rigid_rot_vec_mul)
KUTACC_NOT_BUILT(kutacc_af2_rigid_rot_matmul)
