// Stand-in for <faiss/MetricType.h>; see README.md in this directory.
#pragma once
#include <cstdint>
namespace faiss {
using idx_t = int64_t;
enum MetricType { METRIC_INNER_PRODUCT = 0, METRIC_L2 = 1 };
}  // namespace faiss
