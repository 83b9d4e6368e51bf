"""Observability: metric sinks, the FLOPs model, training log line, profiler switches."""
