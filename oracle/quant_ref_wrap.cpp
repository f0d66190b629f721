// quant_ref_wrap.cpp -- test infrastructure: C entry points around fragments of the REFERENCE's
// quantisation tool, so the restated quantiser (oracle.c) and the product's (csrc/quant.cu) can be pinned
// to reference code.  The fragments are not in this repository: oracle/Makefile cuts them out of
// tools/optimize/model_quant.hpp of the reference tree at build time (sed -n, by line range, each range
// checked against the text it is expected to start with) into oracle/_ref/quant_frag_*.inc, and this file
// only supplies the variables those lines use.  The whole tool cannot be built here (it needs OpenCV and
// the reference's runtime); these pieces have no dependency beyond CONV_CONFIG_S and the C++ library.
//
//   frag_weight  model_quant.hpp:6-29     quant_weight_bias (the whole function)
//   frag_greater :78-81                   the |a| > |b| ordering of the percent method
//   frag_pct2    :159-165                 percent: per-image sort and copy of the largest values
//   frag_pct3    :173-179                 percent: final sort and threshold pick
//   frag_calckl  :187-195                 calc_kl
//   frag_hist    :323-329                 histogram of |x| / max over 2048 bins, zeros skipped
//   frag_kl      :340-431                 KL threshold search
//   frag_max     :526-533                 running max |x|
//   frag_mse     :586-619                 MSE threshold search
//   frag_silulut host/ops/conv.h:180-188  the SiLU table the reference host hands to Conv (inputs[11])
//   frag_gelulut host/ops/gelu.h:82-91    the Gelu table (same header set: "math.h" is included by gelu.h itself)
// The include set is that of the reference's translation unit (tools/optimize/optimize.hpp:3-29,
// common/nn_common.h:4-6, common/utils_cpp.hpp:6-17, host/net.h:6-19) without OpenCV, which is not
// installed here.  It matters which math declarations are visible: optimize.hpp:28 pulls in every operator
// header before model_quant.hpp, and host/ops/gelu.h:5 includes "math.h".  Under g++ that is the C++
// wrapper, which exports the float overloads into the global namespace, so the unqualified fabs / log /
// floor / ceil calls of the quantiser on float arguments are FLOAT functions: the histogram index
// fabs(x) * 2048 * 1.0f / max and the KL sum are evaluated in single precision.  (Without that header
// they would be the C library's double functions and a few histogram counts would move by one bin.)
#include <iostream>
#include <fstream>
#include "cstring"
#include <time.h>
#include <vector>
#include "cmath"
#include "math.h"      // host/ops/gelu.h:5, reached through ops_head.h (optimize.hpp:28)
#include <dlfcn.h>
#include <memory>
#include <sys/time.h>
#include <thread>
#include <pthread.h>
#include <functional>
#include <algorithm>
#include <numeric>
#include "stdint.h"
#include <stdlib.h>
#include <stdio.h>
#include <sstream>
#include <unordered_map>
#include "cctype"
#include <map>
#include <list>
#include <set>
#include <string>

#include "../include/one_abi.h"

#include "_ref/quant_frag_weight.inc"
#include "_ref/quant_frag_greater.inc"
#include "_ref/quant_frag_calckl.inc"

namespace {
// stands in for the reference's extractor: the fragments read operand sizes through it
struct FakeExe {
    std::unordered_map<std::string, BUFFER_INFO_S> operand_buf_map;
};
}  // namespace

extern "C" void ref_quant_weight_bias(CONV_CONFIG_S *cfg, float *weight_in_place, float *bias_in_place, int32_t *weight_shapes)
{
    quant_weight_bias(cfg, weight_in_place, bias_in_place, weight_shapes);
}

// max |x| over one tensor, continuing from `running` (the reference keeps the largest over all images)
extern "C" float ref_abs_max(const float *x, int64_t n, float running)
{
    std::unordered_map<std::string, float> max_elem_map;
    const std::string ifmap_name = "x";
    max_elem_map[ifmap_name] = running;
    float *fmap_ptr = const_cast<float *>(x);
    int64_t elem_size = n;
    {
#include "_ref/quant_frag_max.inc"
    }
    return max_elem_map[ifmap_name];
}

// accumulate one tensor into the 2048-bin histogram
extern "C" void ref_hist_accumulate(const float *x, int64_t n, float max_abs, float *hist2048)
{
    const int32_t num_his_bins = 2048;
    std::unordered_map<std::string, std::vector<float>> his_map;
    const std::string ifmap_name = "x";
    his_map[ifmap_name] = std::vector<float>(hist2048, hist2048 + num_his_bins);
    float cur_ifmap_max = max_abs;
    float *ofmap_ptr = const_cast<float *>(x);
    int64_t elem_size = n;
    {
#include "_ref/quant_frag_hist.inc"
    }
    std::copy(his_map[ifmap_name].begin(), his_map[ifmap_name].end(), hist2048);
}

static float search(const float *hist2048, int32_t elem_count, float max_abs, bool kl)
{
    const int32_t num_his_bins = 2048;
    std::unordered_map<std::string, std::vector<float>> his_map;
    std::unordered_map<std::string, int32_t> elem_size_map;
    std::unordered_map<std::string, float> max_elem_map, threshold_map;
    his_map["x"] = std::vector<float>(hist2048, hist2048 + num_his_bins);
    elem_size_map["x"] = elem_count;
    max_elem_map["x"] = max_abs;
    if (kl) {
        for (auto m_i : his_map) {
#include "_ref/quant_frag_kl.inc"
        }
    } else {
        for (auto m_i : his_map) {
#include "_ref/quant_frag_mse.inc"
        }
    }
    return threshold_map["x"];
}

extern "C" float ref_mse_threshold(const float *hist2048, int32_t elem_count, float max_abs) { return search(hist2048, elem_count, max_abs, false); }
extern "C" float ref_kl_threshold(const float *hist2048, int32_t elem_count, float max_abs) { return search(hist2048, elem_count, max_abs, true); }

// The percent method over n_img tensors of `elem` values each (images[i] points at image i's copy of the
// operand).  The set-up lines of the reference (model_quant.hpp:98, :107, :115-116) are restated here; the
// sorting, copying and the threshold pick are the reference's lines.
extern "C" float ref_percent_threshold(const float *const *images, int32_t n_img, int32_t elem)
{
    FakeExe fake, *exe_net = &fake;
    const std::string ifmap_name = "x";
    exe_net->operand_buf_map[ifmap_name].elem_size = elem;
    std::unordered_map<std::string, float> threshold_map;
    int32_t calibrate_img_num = n_img;
    float percent = 99.998 / 100;
    const int32_t affluence_ratio = 10;
    std::unordered_map<std::string, std::vector<float>> large_elem_map;
    {
        int32_t ifmap_elem_size = elem;
        int32_t mult_batch_large_elem_size = (int32_t)(calibrate_img_num * ifmap_elem_size * (1 - percent) * affluence_ratio);
        large_elem_map[ifmap_name] = std::vector<float>(mult_batch_large_elem_size, 0);
    }
    for (int32_t img_i = 0; img_i < n_img; ++img_i) {
        float *ifmap_ptr = const_cast<float *>(images[img_i]);
        int32_t ifmap_elem_size = elem;
#include "_ref/quant_frag_pct2.inc"
    }
    for (auto map_i : large_elem_map) {
#include "_ref/quant_frag_pct3.inc"
    }
    return threshold_map[ifmap_name];
}

// The activation tables (8192 entries) exactly as the reference host builds them.
extern "C" void ref_silu_lut(float *out8192)
{
    std::vector<float> lut;
    {
#include "_ref/quant_frag_silulut.inc"
    }
    std::copy(lut.begin(), lut.end(), out8192);
}

extern "C" void ref_gelu_lut(float *out8192)
{
    std::vector<float> lut;
    {
#include "_ref/quant_frag_gelulut.inc"
    }
    std::copy(lut.begin(), lut.end(), out8192);
}
