"""The step function, the scheduler above it, and the request API."""
