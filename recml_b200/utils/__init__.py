"""Utilities: dataclass factories, lazy configs and flag parsing."""
from recml_b200.utils import py_utils
from recml_b200.utils import types
from recml_b200.utils.types import (Dataclass, Factory, FactoryProtocol,
                                    FrozenDataclass, ObjectFactory)
from recml_b200.config import (Config, build, select, DEFINE_fiddle_config,
                               FiddleFlag, CallExpression)
from recml_b200 import config
