"""Python half of the runtime layer: lazy init, device/stream/memory/RNG APIs, AMP, serialization."""
