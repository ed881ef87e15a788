/* Stand-in for the CUDA toolkit header of the same name: the reference kernels use only this constant. */
#pragma once
#define CUDART_PI_F 3.141592654f
