"""Parts of a model.  Importing the package registers the built-in kinds."""
from . import attention, feed_forward, model, norm, position  # noqa: F401
