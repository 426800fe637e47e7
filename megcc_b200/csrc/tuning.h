// Kernel-selection switches for experiments and tests. They are read from the MB200_*
// environment variables ONCE, when the library first needs them, and can be changed afterwards
// only through mb200_set_option(): no launch path consults the environment.
#pragma once

namespace mb200 {

struct Tuning {
    int conv_bn = 0;        // MB200_CONV_BN        0 = by shape, 128 or 256 = that tile width
    int conv_pair = 0;      // MB200_CONV_PAIR      1 = 256 x 256 tiles on pairs of SMs
    int conv_splitk = 0;    // MB200_CONV_SPLITK    2..4 = split the last wave's tiles along K
    int wide128 = 1;        // MB200_NO_WIDE128     0 = 64-channel rows even where 128 fit
    int patch_ctas = 0;     // MB200_PATCH_CTAS     1..3 = resident CTAs the patch kernel tries first
    int patch_alone = 0;    // MB200_PATCH_ALONE    1 = patch kernel even with one CTA per SM
    int patch_plain = 0;    // MB200_PATCH_PLAIN    1 = 16-channel planes for 64-channel layers
    int overlap_loads = 1;  // MB200_OVERLAP_LOADS  0 = one 32-column TMEM load per chunk in the halo-patch epilogue
    int dw_tensor = 1;      // MB200_DW_TENSOR      0 = depthwise 3x3/1 on the CUDA cores only
    int dw_out = 0;         // MB200_DW_OUT         2 | 4 = outputs per thread of the depthwise kernel
    int dw_one_output = 0;  // MB200_DW_ONE_OUTPUT  1 = one output per thread
    int fast_requant = 1;   // MB200_NO_FAST_REQUANT  0 = always the reference's float operations
    int debug = 0;          // MB200_DEBUG          1 = one line per launch on stderr
    int pdl = 1;            // MB200_NO_PDL         0 = plain stream-ordered launches
};

Tuning& tuning();

}  // namespace mb200
