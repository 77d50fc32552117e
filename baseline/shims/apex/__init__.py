"""Stand-in for the few apex names the reference imports (apex is not in this image).  The fused
multi-tensor Adam maps onto torch's own fused multi-tensor kernels.  Only used by the reference arm of
bench.py."""
