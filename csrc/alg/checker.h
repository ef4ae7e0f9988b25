// checker.h - static verification of a Schedule, run for every template x rank count in the tests.
//
// It plays every rank's program symbolically (slice contents are multisets of "input slice s of
// rank q") under the POST/WAIT semantics and reports
//   deadlock          some rank still has work but nobody can advance
//   notify imbalance  a slot is left with unconsumed posts, or a wait can never be served
//   memory conflict   two accesses to the same slice, at least one a write, that are not ordered by
//                     the happens-before relation the notifies induce (vector clocks) - the class of
//                     bug the reference's task-DAG checker hunts (test/st/algorithm checker)
//   capacity          a slice is moved into a slice that cannot hold it
//   semantics         the final contents of OUTPUT are not what the collective promises
#pragma once
#include <string>
#include <vector>

#include "ir.h"

namespace hc {

struct CheckOptions {
    bool inPlace = false;   // INPUT and OUTPUT name the same memory (slice i aliases slice i)
    bool checkRaces = true;
};

struct CheckReport {
    bool ok = true;
    std::vector<std::string> errors;
    size_t primsExecuted = 0;
    uint32_t maxStep = 0;
    std::string Summary() const;
};

CheckReport CheckSchedule(const Schedule &s, const CheckOptions &opt = CheckOptions());

}  // namespace hc
