"""Host-side utilities: debug switches, tracing and timing, op traces, dumps, parity checks."""
