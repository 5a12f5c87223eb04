"""Command-line tools: device management (``smi``), device/agent dump (``info``), tracing
launcher (``prof``), trace database (``tracedb``), telemetry daemon (``telemetry``) and roofline
report (``roofline``). Run any of them as ``python -m rocm_systems_b200.tools.<name> --help``."""
