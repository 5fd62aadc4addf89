// Forwarding header: code written against the reference's include tree (#include "operations/kudnn_linear_res.hpp") finds the same
// declarations here; this build keeps them all in kudnn.hpp.
#ifndef KUDNN_B200_FWD_OPERATIONS_KUDNN_LINEAR_RES_HPP
#define KUDNN_B200_FWD_OPERATIONS_KUDNN_LINEAR_RES_HPP
#include "../kudnn.hpp"
#endif
