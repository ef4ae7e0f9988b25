// The device-side primitive library is part of the public interface: include/hcomm_device.cuh.
#pragma once
#include "../../include/hcomm_device.cuh"
