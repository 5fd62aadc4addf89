// Forwarding header: code written against the reference's include tree (#include "types/kudnn_normalization.hpp") finds the same
// declarations here; this build keeps them all in kudnn.hpp.
#ifndef KUDNN_B200_FWD_TYPES_KUDNN_NORMALIZATION_HPP
#define KUDNN_B200_FWD_TYPES_KUDNN_NORMALIZATION_HPP
#include "../kudnn.hpp"
#endif
