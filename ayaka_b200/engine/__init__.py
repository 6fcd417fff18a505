"""The engine: step function, scheduler, request state and the Python entry point."""
