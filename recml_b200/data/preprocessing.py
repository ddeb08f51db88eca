"""Mode flag handed to feature transformations (`recml/core/data/preprocessing.py:19-24`)."""
import enum


class PreprocessingMode(str, enum.Enum):
  """Which phase a preprocessing function is running in."""
  TRAINING = "training"
  EVAL = "eval"
  SERVING = "serving"

  def __str__(self) -> str:
    return self.value
