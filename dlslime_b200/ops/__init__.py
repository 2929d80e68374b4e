"""sm_100a ops: quantisation, tcgen05 GEMMs, NVLink copy, collectives, EP, KV transfer."""
