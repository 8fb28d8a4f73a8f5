"""INT8 stand-alone tools for RWKV-7: offline quantizers, loaders, weight-only (W8A16) projections."""
