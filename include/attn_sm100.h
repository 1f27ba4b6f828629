// C++ face of the sm_100a attention forward for the reference's testbed: the launch functions of
// tk_4090_fwd.hpp:5 / baseline.hpp:5 take `const HostAttnArgs&` (matrix_util.hpp:40-45: stream, N, d and
// device arrays q, k, v of __nv_bfloat16 held by unique_ptr) and a device output pointer.
// `launch_attn_sm100_fwd_kernel` is a template over that argument type, so it can stand where
// `launch_tk_4090_fwd_kernel(args, o)` stands without this header including the reference's.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>

#include "spork_b200.h"

// One head: q, k, v, o are (N, d) row-major bfloat16 on the device; scale 1/sqrt(d) as in
// simple_attn (torch_attn.py:11-16).  Asynchronous on args.stream.
template <class HostAttnArgsT>
inline int launch_attn_sm100_fwd_kernel(const HostAttnArgsT& args, __nv_bfloat16* o)
{
    const int rc = spork_attn_sm100_fwd_bf16(1, args.N, args.d, args.q.get(), args.k.get(), args.v.get(), o,
                                             1.0f / sqrtf((float)args.d), args.stream);
    if (rc != 0) {
        fprintf(stderr, "launch_attn_sm100_fwd_kernel: error %d (N=%d d=%d; d must be 64 or 128)\n", rc, args.N, args.d);
    }
    return rc;
}
