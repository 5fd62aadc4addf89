// Forwarding header: code written against the reference's include tree (#include "service/kudnn_service.hpp") finds the same
// declarations here; this build keeps them all in kudnn.hpp.
#ifndef KUDNN_B200_FWD_SERVICE_KUDNN_SERVICE_HPP
#define KUDNN_B200_FWD_SERVICE_KUDNN_SERVICE_HPP
#include "../kudnn.hpp"
#endif
