"""Measurement: the shapes that are benchmarked (as data), the work a step has to do (bytes and flops), timers
on the device, and the workloads that `bench.py` runs.  The reference keeps the same things in its bench crate and
its bench scripts (crates/bench/src/cert.rs:15-89, crates/backend-hip/src/profile.rs:48-83,
scripts/bench/bench_mixed_sustained.py)."""
