// ops/blas.hpp -- BLAS facade so that engine.blas().gemm(...) resolves (reference:
// include/SushiBLAS/ops/blas.hpp:49-57, which also inherits Level1, Level2 and SparseBLAS;
// those families are outside the fp32 GEMM path and are not part of this build).
#pragma once

#include <SushiBLAS/ops/blas/level3.hpp>

namespace SushiBLAS
{
    class Engine;

    class BLASOps : public Level3
    {
        public:
            explicit BLASOps(Engine& e) : Level3(e) {}
    };
} // namespace SushiBLAS
