// Stand-in for SwiftWare-Lab/benchmark "Stats.h": the inspectors only write
// into the OtherStats map.
#ifndef ORACLE_SHIM_STATS_H
#define ORACLE_SHIM_STATS_H
#include <map>
#include <string>
#include <vector>
namespace swiftware { namespace benchmark {
struct Stats {
  std::map<std::string, std::vector<double>> OtherStats;
};
}} // namespace swiftware::benchmark
#endif
