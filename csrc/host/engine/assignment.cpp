#include "engine/assignment.h"

namespace slime {

void split_assign_by_max_length(const AssignmentBatch& in, AssignmentBatch& out, size_t max_length)
{
    if (max_length == 0) {
        out.insert(out.end(), in.begin(), in.end());
        return;
    }
    size_t pieces = 0;
    for (const auto& a : in) pieces += a.length <= max_length ? 1 : (a.length + max_length - 1) / max_length;
    out.reserve(out.size() + pieces);
    for (const auto& a : in) {
        if (a.length <= max_length) {
            out.push_back(a);
            continue;
        }
        for (uint64_t done = 0; done < a.length; done += max_length) {
            const uint64_t n = std::min<uint64_t>(max_length, a.length - done);
            out.emplace_back(a.mr_key, a.remote_mr_key, a.target_offset + done, a.source_offset + done, n);
        }
    }
}

void split_assign_by_step(const AssignmentBatch& in, std::vector<AssignmentBatch>& out, size_t step)
{
    if (in.empty() || step == 0) return;
    out.reserve(out.size() + (in.size() + step - 1) / step);
    for (size_t i = 0; i < in.size(); i += step) {
        const size_t n = std::min(step, in.size() - i);
        out.emplace_back(in.begin() + i, in.begin() + i + n);
    }
}

void nsplit_assign_by_step(const AssignmentBatch& in, std::vector<AssignmentBatch>& out, size_t nstep)
{
    if (nstep == 0) return;
    split_assign_by_step(in, out, (in.size() + nstep - 1) / nstep);
}

}  // namespace slime
