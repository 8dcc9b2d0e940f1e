// Stand-in for the reference's utils/utils.hpp umbrella header: pulls in only
// the two real headers its kernel templates need (xprintf, one<half>/zero<half>).
#pragma once
#include "utils/debug.hpp"
#include "utils/cuda_helpers.cuh"
