"""Execution session, runner switches and byte model for the decode step
(reference: ``benchmarks/cudagraph.py``, ``benchmarks/runner.py``, ``benchmarks/bytes.py``)."""
