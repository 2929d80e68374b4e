// `nanoctrl obs`: reads the snapshots that ObsReporters publish under {scope:}obs:peer:* and prints
// them as tables (or JSON). A snapshot is "stopped" when it says so, "stale" when older than
// --stale-ms, else "alive" (the rule of the reference's viewer, NanoCtrl/src/obs.rs:253-266 in the reference).
#pragma once

#include <string>
#include <vector>

#include "core/json.hpp"

namespace slime {
namespace ctrl {

struct PeerSnapshot {
    std::string alias, state;
    int64_t     age_ms = 0;
    Json        data;
};

std::string snapshot_state(const Json& snap, int64_t now_ms, int64_t stale_ms);
std::string human_bps(double bits_per_second);
std::string human_bytes(double bytes);
// Renders one view ("status" | "peers" | "nics" | "links") of the parsed snapshots.
std::string render_obs_view(const std::vector<PeerSnapshot>& peers, const std::string& view, bool as_json);
// Fetches the snapshots from a RESP server at host:port (or redis://host:port).
std::vector<PeerSnapshot> fetch_snapshots(const std::string& address, const std::string& scope, int64_t stale_ms);
int obs_view_main(const std::string& address, const std::string& scope, const std::string& view, int64_t stale_ms, bool as_json);

}  // namespace ctrl
}  // namespace slime
