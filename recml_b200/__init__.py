"""recml_b200: a Blackwell-native recommender training and serving framework.

Public surface (the names exported by the reference's `recml/__init__.py:19-40`).
"""
from recml_b200 import config
from recml_b200 import data
from recml_b200 import embedding
from recml_b200 import layers
from recml_b200 import metrics
from recml_b200 import utils
from recml_b200.metrics.base import Metric
from recml_b200.training.core import Experiment, Trainer as TrainerInterface, run_experiment
from recml_b200.training.optim_factory import (AdagradFactory, AdamFactory, OptimizerFactory,
                                               SGDFactory)
from recml_b200.training.partitioning import (DataParallelPartitioner, ModelParallelPartitioner,
                                              NullPartitioner, Partitioner)
from recml_b200.training.state import JaxState, KerasState, State
from recml_b200.training.task import JaxTask, Task
from recml_b200.training.trainer import JaxTrainer, Trainer
from recml_b200.training.module_trainer import KerasTask, KerasTrainer, ModuleTask, ModuleTrainer
from recml_b200.utils.types import Factory, FactoryProtocol, ObjectFactory

__version__ = "0.1.0"
