"""Distributed layer: meshes, placements, collective plans, rendezvous, transports, fused reducers."""
