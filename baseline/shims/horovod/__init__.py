"""Stand-in for the Horovod package, used only by the reference arm of bench.py."""
