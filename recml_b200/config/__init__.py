"""Lazy configuration graph + the `config:/fiddler:/set:` command-line flag."""
from recml_b200.config.lazy import Config, Selection, build, select, set_path
from recml_b200.config.flags import CallExpression, DEFINE_fiddle_config, FiddleFlag
