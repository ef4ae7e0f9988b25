// The layout shared by the host runtime and device code is part of the public interface: include/hcomm_comm_dev.h.
#pragma once
#include "../../include/hcomm_comm_dev.h"
