"""No-op stand-in for ``matplotlib`` (the reference's tools/utils/plotting.py draws latency plots with it).  Test
infrastructure: put on ``sys.path`` only when the real package is not installed."""
