// Forwarding header: code written against the reference's include tree (#include "operations/kudnn_gemm.hpp") finds the same
// declarations here; this build keeps them all in kudnn.hpp.
#ifndef KUDNN_B200_FWD_OPERATIONS_KUDNN_GEMM_HPP
#define KUDNN_B200_FWD_OPERATIONS_KUDNN_GEMM_HPP
#include "../kudnn.hpp"
#endif
