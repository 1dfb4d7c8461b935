"""Parallelism strategies built on the collectives: data, tensor/sequence and expert parallel."""
