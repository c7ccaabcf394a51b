"""KV geometry of a slot, the fp8 block codec oracle, and the HBM / pinned-host chunk tiers."""
