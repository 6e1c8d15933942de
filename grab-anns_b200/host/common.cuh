// Stand-in for the reference's src/index/common.cuh (the device the library runs on).
#pragma once
#ifndef CUDA_DEVICE_ID
#define CUDA_DEVICE_ID 0
#endif
