"""Host oracle of the attention path — test infrastructure, never part of the product path."""
