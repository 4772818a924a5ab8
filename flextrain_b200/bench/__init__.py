"""Benchmarks and the loss-curve parity harness: ``parity`` (engine against a naive autograd model under forced working
sets), ``naive`` (that model), ``kernel_cases`` / ``comm_cases`` (one kernel or one fused collective path at a time).
Nothing is imported here: ``python -m flextrain_b200.bench.<module>`` keeps its start-up light."""
