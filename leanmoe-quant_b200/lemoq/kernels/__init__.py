"""Decode-path ops (same module names and signatures as the reference's ``lemoq.kernels``)."""
