"""CPU oracle of the talker token loop: test infrastructure, never on the product path."""
