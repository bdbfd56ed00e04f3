"""Drop-in mirror of the reference's ``core`` modules that sit on the inference
hot path.  Names, argument order, defaults and return types follow the
reference; the arithmetic runs in ``libeoq_b200.so`` on the GPU."""
