"""Synthetic workloads of the paged KV-cache path, one per benchmark configuration.

The counterpart of the reference's ``python/barqtrain/benchmarks`` package for this path: the
reference ships only a training benchmark there and measures the cache through a notebook; these
are the append / gather / churn workloads its configurations describe, on seeded synthetic data.
"""
