// SushiBLAS.h -- master header (reference: include/SushiBLAS/SushiBLAS.h:41-45).
#pragma once

#include "core/common.hpp"
#include "core/logger.hpp"
#include "storage.hpp"
#include "tensor.hpp"
#include "engine.hpp"
