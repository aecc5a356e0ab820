"""Image inputs for multimodal models: preprocessing, placeholder expansion, embedding merge, attention masks."""
from .utils import bidirectional_block_mask, expand_image_placeholders, merge_mm_embeddings  # noqa: F401
from .processor import preprocess_images  # noqa: F401
