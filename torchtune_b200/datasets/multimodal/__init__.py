from ._builders import TheCauldronToMessages, llava_instruct_dataset, multimodal_chat_dataset, the_cauldron_dataset, the_cauldron_transform, vqa_dataset

__all__ = ["TheCauldronToMessages", "llava_instruct_dataset", "multimodal_chat_dataset", "the_cauldron_dataset", "the_cauldron_transform", "vqa_dataset"]
