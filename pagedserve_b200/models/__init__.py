"""Architectures: importing this package registers the built-in ones."""

from pagedserve_b200.models import gpt2  # noqa: F401  (registers "GPT2LMHeadModel")
from pagedserve_b200.models import tefopel  # noqa: F401  (registers "Tefopel")
from pagedserve_b200.models import gozunex  # noqa: F401  (registers "Gozunex")
from pagedserve_b200.models import zositar  # noqa: F401  (registers "Zositar")
from pagedserve_b200.models import pagatar  # noqa: F401  (registers "Pagatar")
from pagedserve_b200.models.model import Model, init_plan  # noqa: F401
from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry  # noqa: F401
