"""Compiler: annotated FX graph -> training DAG -> directive rewrites -> per-device plans."""
