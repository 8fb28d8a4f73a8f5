"""INT4 weight-only (W4A16) tools for RWKV-7: offline quantizers, loaders, projections."""
