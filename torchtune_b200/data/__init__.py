from ._collate import (
    left_pad_sequence,
    padded_collate,
    padded_collate_dpo,
    padded_collate_packed,
    padded_collate_sft,
    padded_collate_tiled_images_and_mask,
)
from ._common import CROSS_ENTROPY_IGNORE_IDX
from ._messages import (
    AlpacaToMessages,
    ChosenRejectedToMessages,
    InputOutputToMessages,
    MaskingStrategy,
    Message,
    OpenAIToMessages,
    Role,
    ShareGPTToMessages,
    mask_messages,
    validate_messages,
)
from ._prompt_templates import (
    ChatMLTemplate,
    GrammarErrorCorrectionTemplate,
    PromptTemplate,
    PromptTemplateInterface,
    QuestionAnswerTemplate,
    SummarizeTemplate,
)
from ._utils import format_content_with_images, load_image, truncate

__all__ = [
    "CROSS_ENTROPY_IGNORE_IDX",
    "GrammarErrorCorrectionTemplate",
    "SummarizeTemplate",
    "OpenAIToMessages",
    "ShareGPTToMessages",
    "AlpacaToMessages",
    "truncate",
    "Message",
    "MaskingStrategy",
    "validate_messages",
    "mask_messages",
    "Role",
    "format_content_with_images",
    "PromptTemplateInterface",
    "PromptTemplate",
    "InputOutputToMessages",
    "ChosenRejectedToMessages",
    "QuestionAnswerTemplate",
    "ChatMLTemplate",
    "padded_collate_sft",
    "padded_collate_dpo",
    "left_pad_sequence",
    "padded_collate",
    "padded_collate_tiled_images_and_mask",
    "padded_collate_packed",
    "load_image",
]
