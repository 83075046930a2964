"""Per-process runtime: rank layout, parameter storage, DAG executor, actor, launcher, health monitoring."""
