"""Ternary formats and linears: the surface of the reference's ``boilerplate/ternary`` package that the hot path uses."""
