"""Measurement and operations tooling around the service: bandwidth sweep and tuner
(``sweep``), tables and curves from its CSV (``report``), per-stage latency of a small
collective (``latency``), co-located tenants under QoS (``multi_tenant``), the multi-job
launcher (``launcher``), QoS window planning (``qos_intervals``), a small case of one
kernel for a profiler (``profile_case``) and timing / clock-sampling helpers (``timing``)."""
