// placeholder until the tensor-core kernels arrive
#pragma once
