"""Model export and batch inference.

The reference's trainers end with `task.export_model(state, model_dir)` (`recml/core/training/
jax_trainer.py:376-382,843-845`; the Keras trainer saves `model.keras`, `keras_trainer.py:99`) and leave
serving to whatever loads that artefact.  Here `export` writes a self-describing directory (weights in the
checkpoint format, tables still sharded so that no rank ever holds a whole 100 GB table, the embedding spec
side-car, and the recipe to rebuild the module) and `load` / `Predictor` bring it up on any number of GPUs
for forward-only use.
"""
from recml_b200.serving.export import Predictor, batch_inference, export, load

__all__ = ["export", "load", "Predictor", "batch_inference"]
