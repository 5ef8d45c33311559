"""`cerium` as the reference's drivers import it, served by cerium_b200.

Put this directory (cerium_b200/as_cerium) on PYTHONPATH and a driver written against the reference's
runtime - ``import cerium.runtime as runtime`` (examples/common.py:91, benchmarks/bootstrap_32K/
bootstrap_runner.py:22) - runs on this library without an edit.  Only the runtime half exists here:
``cerium.dsl`` and ``cerium.compiler`` are the reference's own (programs are compiled by its compiler).
"""
