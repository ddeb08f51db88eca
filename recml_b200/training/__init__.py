"""Training runtime: trainer contract, trainers, state, optimizers, partitioners."""
