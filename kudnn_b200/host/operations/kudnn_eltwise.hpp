// Forwarding header: code written against the reference's include tree (#include "operations/kudnn_eltwise.hpp") finds the same
// declarations here; this build keeps them all in kudnn.hpp.
#ifndef KUDNN_B200_FWD_OPERATIONS_KUDNN_ELTWISE_HPP
#define KUDNN_B200_FWD_OPERATIONS_KUDNN_ELTWISE_HPP
#include "../kudnn.hpp"
#endif
