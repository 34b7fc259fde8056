#pragma once
#define GERN_ROOT_DIR "/root/reference"
#define GERN_CUDA_ARCH ""
